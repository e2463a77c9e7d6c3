// mmt4d on HOST buffers: the reference's call shape (host pointers in, host pointer out) served
// by the device kernels, with the transfers pipelined against the computation.
//
// The work is cut into jobs, each a block of LHS tile rows times a chunk of RHS tile rows.
// Three internal streams per device run as a pipeline: H copies operands to the device, S runs
// mmt4d on one job after another (through iree_uk_b200_mmt4d_ws, so the tensor-core kernels
// are used), C copies each job's output slab back to the host with a 2-D copy into the
// caller's [M][N][M0][N0] layout. The device-to-host stream is the long pole (the f32/i32
// output is the largest buffer), so the schedule is built to start it early and keep it busy:
// the RHS chunks grow geometrically from a small first one, and the first chunk is computed in
// several blocks of LHS tile rows, each as soon as that block of the LHS has arrived, so that
// the first output leaves after a fraction of the LHS upload instead of all of it.
//
// All device memory comes from the caller's arena; the three streams and the events are
// host-side objects created once per device.
#include <algorithm>
#include <mutex>

#include "uk_common.h"

namespace uk {
namespace {

constexpr int kMaxChunks = 8;      // chunks of RHS tile rows
constexpr int kLhsBlocks = 4;      // blocks of LHS tile rows (used by the first RHS chunk)
constexpr int kMaxJobs = kMaxChunks + kLhsBlocks;

struct HostPipe {
  bool ready = false;
  std::mutex enqueue;  // one call at a time builds its chain of copies, kernels and events
  cudaStream_t h2d = nullptr, compute = nullptr, d2h = nullptr;
  cudaEvent_t start = nullptr, lhs_done = nullptr, done = nullptr;
  cudaEvent_t in_done[kMaxChunks] = {}, lhs_block_done[kLhsBlocks] = {}, out_ready[kMaxJobs] = {};
};

HostPipe* host_pipe() {
  constexpr int kMaxDevices = 64;
  static HostPipe pipes[kMaxDevices];
  static std::mutex mu;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  HostPipe& p = pipes[dev];
  if (!p.ready) {
    bool ok = cudaStreamCreateWithFlags(&p.h2d, cudaStreamNonBlocking) == cudaSuccess &&
              cudaStreamCreateWithFlags(&p.compute, cudaStreamNonBlocking) == cudaSuccess &&
              cudaStreamCreateWithFlags(&p.d2h, cudaStreamNonBlocking) == cudaSuccess;
    auto ev = [&](cudaEvent_t* e) {
      ok = ok && cudaEventCreateWithFlags(e, cudaEventDisableTiming) == cudaSuccess;
    };
    ev(&p.start); ev(&p.lhs_done); ev(&p.done);
    for (int i = 0; i < kMaxChunks; ++i) ev(&p.in_done[i]);
    for (int i = 0; i < kLhsBlocks; ++i) ev(&p.lhs_block_done[i]);
    for (int i = 0; i < kMaxJobs; ++i) ev(&p.out_ready[i]);
    if (!ok) return nullptr;
    p.ready = true;
  }
  return &p;
}

int64_t round_up(int64_t v, int64_t q) { return (v + q - 1) / q * q; }

struct Chunk {
  int64_t begin, count;
};

// Split of N tile rows into at most kMaxChunks contiguous chunks of 4, 1, 2, 4, 5, 8, 8
// thirty-seconds of N. The first chunk is computed block by block of the LHS while the LHS is
// still arriving, so it is sized to keep the device-to-host copies busy for about as long as
// the LHS upload takes; the next ones start small (their RHS rows must arrive before the
// copies run dry) and grow, which keeps the per-call overhead low.
int make_chunks(int64_t N, Chunk* out) {
  static const int kWeights[kMaxChunks] = {4, 1, 2, 4, 5, 8, 8, 0};
  int n = 0;
  if (N < 64) {  // too few rows to grade: equal chunks
    n = int(std::min<int64_t>(kMaxChunks, std::max<int64_t>(N, 1)));
    const int64_t base = N / n, rem = N % n;
    int64_t b = 0;
    for (int i = 0; i < n; ++i) {
      out[i].begin = b;
      out[i].count = base + (i < rem ? 1 : 0);
      b += out[i].count;
    }
    return n;
  }
  int64_t b = 0;
  for (int i = 0; i < kMaxChunks && b < N; ++i) {
    int64_t c = kWeights[i] ? N * kWeights[i] / 32 : N - b;
    if (i == kMaxChunks - 1 || kWeights[i + 1] == 0) c = N - b;  // the last one takes the rest
    c = std::min(c, N - b);
    out[n].begin = b;
    out[n].count = c;
    b += c;
    ++n;
  }
  return n;
}

// Contiguous, near-equal split of M tile rows into at most kLhsBlocks blocks.
int make_lhs_blocks(int64_t M, Chunk* out) {
  const int n = int(std::min<int64_t>(kLhsBlocks, std::max<int64_t>(M, 1)));
  const int64_t base = M / n, rem = M % n;
  int64_t b = 0;
  for (int i = 0; i < n; ++i) {
    out[i].begin = b;
    out[i].count = base + (i < rem ? 1 : 0);
    b += out[i].count;
  }
  return n;
}

struct ArenaLayout {
  int64_t lhs_bytes, rhs_bytes, out_bytes, ws_bytes, total;
  int64_t lhs_row_bytes, rhs_row_bytes;  // tight bytes of one tile row
  int64_t out_tile_bytes;                // bytes of one M0 x N0 output tile
};

bool arena_layout(const iree_uk_mmt4d_params_t* p, ArenaLayout* a) {
  Mmt4dTypes t;
  if (!mmt4d_types(p->flags, &t)) return false;
  const int lb = elem_bits(t.lhs), rb = elem_bits(t.rhs), ob = elem_bits(t.out);
  a->lhs_row_bytes = p->K * p->M0 * p->K0 * lb / 8;
  a->rhs_row_bytes = p->K * p->N0 * p->K0 * rb / 8;
  a->out_tile_bytes = int64_t(p->M0) * p->N0 * ob / 8;
  // Tile rows are stored tight on the device, each padded to 16 bytes so that every chunk
  // stays aligned for the vector and TMA paths.
  a->lhs_row_bytes = round_up(a->lhs_row_bytes, 16);
  a->rhs_row_bytes = round_up(a->rhs_row_bytes, 16);
  a->lhs_bytes = round_up(p->M * a->lhs_row_bytes, 1024);
  a->rhs_bytes = round_up(p->N * a->rhs_row_bytes, 1024);
  a->out_bytes = round_up(p->M * p->N * a->out_tile_bytes, 1024);
  // workspace of the largest job (all LHS tile rows x the largest chunk)
  Chunk ch[kMaxChunks];
  const int nch = make_chunks(p->N, ch);
  iree_uk_mmt4d_params_t q = *p;
  q.N = 0;
  for (int i = 0; i < nch; ++i) q.N = std::max<int64_t>(q.N, ch[i].count);
  a->ws_bytes = round_up(int64_t(mmt4d_tc_workspace_size(&q)), 1024);
  a->total = a->lhs_bytes + a->rhs_bytes + a->out_bytes + a->ws_bytes;
  return true;
}

}  // namespace
}  // namespace uk

using namespace uk;

extern "C" {

size_t iree_uk_b200_mmt4d_host_arena_size(const iree_uk_mmt4d_params_t* params) {
  if (!params || validate_mmt4d(params)) return 0;
  ArenaLayout a;
  if (!arena_layout(params, &a)) return 0;
  return size_t(a.total);
}

namespace {
int mmt4d_host_impl(const iree_uk_mmt4d_params_t* params, const void* device_lhs,
                    iree_uk_index_t device_lhs_stride0, void* device_arena, size_t arena_bytes,
                    void* cu_stream);
}  // namespace

int iree_uk_b200_mmt4d_host(const iree_uk_mmt4d_params_t* params, void* device_arena,
                            size_t arena_bytes, void* cu_stream) {
  return mmt4d_host_impl(params, nullptr, 0, device_arena, arena_bytes, cu_stream);
}

int iree_uk_b200_mmt4d_host_resident_lhs(const iree_uk_mmt4d_params_t* params,
                                         const void* device_lhs,
                                         iree_uk_index_t device_lhs_stride0, void* device_arena,
                                         size_t arena_bytes, void* cu_stream) {
  if (!device_lhs || device_lhs_stride0 < 0) return IREE_UK_B200_INVALID_ARGUMENT;
  return mmt4d_host_impl(params, device_lhs, device_lhs_stride0, device_arena, arena_bytes,
                         cu_stream);
}

}  // extern "C"

namespace {
int mmt4d_host_impl(const iree_uk_mmt4d_params_t* params, const void* device_lhs,
                    iree_uk_index_t device_lhs_stride0, void* device_arena, size_t arena_bytes,
                    void* cu_stream) {
  const int rc = validate_mmt4d(params);
  if (rc) return rc;
  const iree_uk_mmt4d_params_t& p = *params;
  const bool acc = (p.flags & IREE_UK_FLAG_MMT4D_ACCUMULATE) != 0;
  if (p.M == 0 || p.N == 0 || (p.K == 0 && acc) || p.M0 == 0 || p.N0 == 0) return IREE_UK_B200_OK;
  ArenaLayout a;
  if (!arena_layout(params, &a)) return IREE_UK_B200_INVALID_ARGUMENT;
  if (!device_arena || arena_bytes < size_t(a.total)) return IREE_UK_B200_WORKSPACE_TOO_SMALL;
  if (reinterpret_cast<uintptr_t>(device_arena) & 255) return IREE_UK_B200_INVALID_ARGUMENT;
  HostPipe* pipe = host_pipe();
  if (!pipe) return IREE_UK_B200_CUDA_ERROR;
  // The three streams and their events belong to the device, so calls from several host
  // threads take turns enqueueing (the work itself is ordered by the streams).
  std::lock_guard<std::mutex> enqueue_lock(pipe->enqueue);
  cudaStream_t user = static_cast<cudaStream_t>(cu_stream);

  Mmt4dTypes t;
  mmt4d_types(p.flags, &t);
  const int lb = elem_bits(t.lhs), rb = elem_bits(t.rhs), ob = elem_bits(t.out);
  char* d_lhs = static_cast<char*>(device_arena);
  char* d_rhs = d_lhs + a.lhs_bytes;
  char* d_out = d_rhs + a.rhs_bytes;
  char* d_ws = d_out + a.out_bytes;
  const char* h_lhs = static_cast<const char*>(p.lhs_buffer) + p.lhs_offset * lb / 8;
  const char* h_rhs = static_cast<const char*>(p.rhs_buffer) + p.rhs_offset * rb / 8;
  char* h_out = static_cast<char*>(p.out_buffer) + p.out_offset * (ob / 8);
  const int64_t h_lhs_pitch = p.lhs_stride0 * lb / 8, h_rhs_pitch = p.rhs_stride0 * rb / 8;
  const int64_t h_out_pitch = p.out_stride0 * (ob / 8);
  const int64_t lhs_w = p.K * p.M0 * p.K0 * lb / 8, rhs_w = p.K * p.N0 * p.K0 * rb / 8;

#define UK_CUDA(x) do { if ((x) != cudaSuccess) return IREE_UK_B200_CUDA_ERROR; } while (0)
  // order the pipeline after what is already enqueued on the caller's stream
  UK_CUDA(cudaEventRecord(pipe->start, user));
  UK_CUDA(cudaStreamWaitEvent(pipe->h2d, pipe->start, 0));
  UK_CUDA(cudaStreamWaitEvent(pipe->compute, pipe->start, 0));
  UK_CUDA(cudaStreamWaitEvent(pipe->d2h, pipe->start, 0));

  Chunk ch[kMaxChunks], lb_[kLhsBlocks];
  const int nch = make_chunks(p.N, ch);
  // With the LHS already on the device there is nothing to upload block by block: one block.
  int nlb = make_lhs_blocks(p.M, lb_);
  if (device_lhs) {
    nlb = 1;
    lb_[0].begin = 0;
    lb_[0].count = p.M;
  }
  const char* d_lhs_rows = device_lhs ? static_cast<const char*>(device_lhs) : d_lhs;
  const int64_t d_lhs_row_bytes = device_lhs ? device_lhs_stride0 * lb / 8 : a.lhs_row_bytes;
  auto upload_lhs_block = [&](int i) -> bool {
    if (!device_lhs && lhs_w > 0 &&
        cudaMemcpy2DAsync(d_lhs + lb_[i].begin * a.lhs_row_bytes, size_t(a.lhs_row_bytes),
                          h_lhs + lb_[i].begin * h_lhs_pitch, size_t(h_lhs_pitch), size_t(lhs_w),
                          size_t(lb_[i].count), cudaMemcpyHostToDevice, pipe->h2d) != cudaSuccess)
      return false;
    return cudaEventRecord(pipe->lhs_block_done[i], pipe->h2d) == cudaSuccess;
  };
  int64_t slab_off = 0;  // device output: one slab [rows][count][M0*N0] per job, back to back
  int job = 0;
  // One job: LHS tile rows [mb, mb + mc) x RHS chunk c. Its inputs are on the device once the
  // events the compute stream has been told to wait for have fired.
  auto run_job = [&](const Chunk& c, int64_t mb, int64_t mc) -> int {
    char* d_slab = d_out + slab_off;
    const int64_t slab_row = c.count * a.out_tile_bytes;  // bytes of one tile row of the slab
    char* h_dst = h_out + mb * h_out_pitch + c.begin * a.out_tile_bytes;
    if (acc) {  // the old output tiles of this job
      if (cudaMemcpy2DAsync(d_slab, size_t(slab_row), h_dst, size_t(h_out_pitch), size_t(slab_row),
                            size_t(mc), cudaMemcpyHostToDevice, pipe->h2d) != cudaSuccess ||
          cudaEventRecord(pipe->out_ready[job], pipe->h2d) != cudaSuccess ||
          cudaStreamWaitEvent(pipe->compute, pipe->out_ready[job], 0) != cudaSuccess)
        return IREE_UK_B200_CUDA_ERROR;
    }
    iree_uk_mmt4d_params_t q = p;
    q.lhs_buffer = d_lhs_rows + mb * d_lhs_row_bytes; q.lhs_offset = 0; q.lhs_stride0 = d_lhs_row_bytes * 8 / lb;
    q.rhs_buffer = d_rhs + c.begin * a.rhs_row_bytes; q.rhs_offset = 0; q.rhs_stride0 = a.rhs_row_bytes * 8 / rb;
    q.out_buffer = d_slab; q.out_offset = 0; q.out_stride0 = c.count * int64_t(p.M0) * p.N0;
    q.M = mc;
    q.N = c.count;
    const int krc = iree_uk_b200_mmt4d_ws(&q, d_ws, size_t(a.ws_bytes), pipe->compute);
    if (krc) return krc;
    if (cudaEventRecord(pipe->out_ready[job], pipe->compute) != cudaSuccess ||
        cudaStreamWaitEvent(pipe->d2h, pipe->out_ready[job], 0) != cudaSuccess ||
        cudaMemcpy2DAsync(h_dst, size_t(h_out_pitch), d_slab, size_t(slab_row), size_t(slab_row),
                          size_t(mc), cudaMemcpyDeviceToHost, pipe->d2h) != cudaSuccess)
      return IREE_UK_B200_CUDA_ERROR;
    slab_off += mc * slab_row;
    ++job;
    return IREE_UK_B200_OK;
  };
  auto upload_rhs_chunk = [&](int j) -> bool {
    if (rhs_w > 0 &&
        cudaMemcpy2DAsync(d_rhs + ch[j].begin * a.rhs_row_bytes, size_t(a.rhs_row_bytes),
                          h_rhs + ch[j].begin * h_rhs_pitch, size_t(h_rhs_pitch), size_t(rhs_w),
                          size_t(ch[j].count), cudaMemcpyHostToDevice, pipe->h2d) != cudaSuccess)
      return false;
    return cudaEventRecord(pipe->in_done[j], pipe->h2d) == cudaSuccess &&
           cudaStreamWaitEvent(pipe->compute, pipe->in_done[j], 0) == cudaSuccess;
  };

  // First RHS chunk: one job per LHS block, each as soon as that block has arrived.
  if (!upload_lhs_block(0) || !upload_rhs_chunk(0)) return IREE_UK_B200_CUDA_ERROR;
  for (int i = 0; i < nlb; ++i) {
    if (i > 0 && !upload_lhs_block(i)) return IREE_UK_B200_CUDA_ERROR;
    UK_CUDA(cudaStreamWaitEvent(pipe->compute, pipe->lhs_block_done[i], 0));
    if (ch[0].count > 0) {
      const int krc = run_job(ch[0], lb_[i].begin, lb_[i].count);
      if (krc) return krc;
    }
  }
  // Remaining chunks: all LHS tile rows at once.
  for (int j = 1; j < nch; ++j) {
    if (ch[j].count == 0) continue;
    if (!upload_rhs_chunk(j)) return IREE_UK_B200_CUDA_ERROR;
    const int krc = run_job(ch[j], 0, p.M);
    if (krc) return krc;
  }
  // the caller's stream completes when the last slab is on the host
  UK_CUDA(cudaEventRecord(pipe->done, pipe->d2h));
  UK_CUDA(cudaStreamWaitEvent(user, pipe->done, 0));
#undef UK_CUDA
  return IREE_UK_B200_OK;
}
}  // namespace
