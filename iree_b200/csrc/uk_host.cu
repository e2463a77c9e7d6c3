// mmt4d on HOST buffers: the reference's call shape (host pointers in, host pointer out) served
// by the device kernels, with the transfers pipelined against the computation.
//
// The RHS tile rows (N) are cut into chunks. Three internal streams per device run as a
// pipeline: H copies the LHS once and then RHS chunk j to the device, S runs mmt4d on chunk j
// (through iree_uk_b200_mmt4d_ws, so the tensor-core kernels are used), C copies output slab j
// back to the host with a 2-D copy into the caller's [M][N][M0][N0] layout. The device-to-host
// stream is the long pole (the f32/i32 output is the largest buffer), so it starts as soon as
// the first chunk is done and then runs back to back while H and S stay ahead of it.
//
// All device memory comes from the caller's arena; the three streams and the events are
// host-side objects created once per device.
#include <algorithm>
#include <mutex>

#include "uk_common.h"

namespace uk {
namespace {

constexpr int kMaxChunks = 8;

struct HostPipe {
  bool ready = false;
  cudaStream_t h2d = nullptr, compute = nullptr, d2h = nullptr;
  cudaEvent_t start = nullptr, lhs_done = nullptr, done = nullptr;
  cudaEvent_t in_done[kMaxChunks] = {}, out_ready[kMaxChunks] = {};
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
    for (int i = 0; i < kMaxChunks; ++i) { ev(&p.in_done[i]); ev(&p.out_ready[i]); }
    if (!ok) return nullptr;
    p.ready = true;
  }
  return &p;
}

int64_t round_up(int64_t v, int64_t q) { return (v + q - 1) / q * q; }

struct Chunk {
  int64_t begin, count;
};

// Contiguous split of N tile rows into at most kMaxChunks chunks.
int make_chunks(int64_t N, Chunk* out) {
  const int n = int(std::min<int64_t>(kMaxChunks, std::max<int64_t>(N, 1)));
  const int64_t base = N / n, rem = N % n;
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
  // workspace of the largest chunk
  Chunk ch[kMaxChunks];
  make_chunks(p->N, ch);
  iree_uk_mmt4d_params_t q = *p;
  q.N = ch[0].count;
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

int iree_uk_b200_mmt4d_host(const iree_uk_mmt4d_params_t* params, void* device_arena,
                            size_t arena_bytes, void* cu_stream) {
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

  if (lhs_w > 0)
    UK_CUDA(cudaMemcpy2DAsync(d_lhs, size_t(a.lhs_row_bytes), h_lhs, size_t(h_lhs_pitch),
                              size_t(lhs_w), size_t(p.M), cudaMemcpyHostToDevice, pipe->h2d));
  UK_CUDA(cudaEventRecord(pipe->lhs_done, pipe->h2d));
  UK_CUDA(cudaStreamWaitEvent(pipe->compute, pipe->lhs_done, 0));

  Chunk ch[kMaxChunks];
  const int nch = make_chunks(p.N, ch);
  int64_t slab_off = 0;  // device output: chunk slabs [M][count][M0*N0], one after another
  for (int j = 0; j < nch; ++j) {
    const Chunk c = ch[j];
    if (c.count == 0) continue;
    char* d_rhs_j = d_rhs + c.begin * a.rhs_row_bytes;
    char* d_slab = d_out + slab_off;
    const int64_t slab_row = c.count * a.out_tile_bytes;  // bytes of one tile row of the slab
    if (rhs_w > 0)
      UK_CUDA(cudaMemcpy2DAsync(d_rhs_j, size_t(a.rhs_row_bytes), h_rhs + c.begin * h_rhs_pitch,
                                size_t(h_rhs_pitch), size_t(rhs_w), size_t(c.count),
                                cudaMemcpyHostToDevice, pipe->h2d));
    if (acc)  // the old output tiles of this chunk
      UK_CUDA(cudaMemcpy2DAsync(d_slab, size_t(slab_row), h_out + c.begin * a.out_tile_bytes,
                                size_t(h_out_pitch), size_t(slab_row), size_t(p.M),
                                cudaMemcpyHostToDevice, pipe->h2d));
    UK_CUDA(cudaEventRecord(pipe->in_done[j], pipe->h2d));
    UK_CUDA(cudaStreamWaitEvent(pipe->compute, pipe->in_done[j], 0));

    iree_uk_mmt4d_params_t q = p;
    q.lhs_buffer = d_lhs; q.lhs_offset = 0; q.lhs_stride0 = a.lhs_row_bytes * 8 / lb;
    q.rhs_buffer = d_rhs_j; q.rhs_offset = 0; q.rhs_stride0 = a.rhs_row_bytes * 8 / rb;
    q.out_buffer = d_slab; q.out_offset = 0; q.out_stride0 = c.count * int64_t(p.M0) * p.N0;
    q.N = c.count;
    const int krc = iree_uk_b200_mmt4d_ws(&q, d_ws, size_t(a.ws_bytes), pipe->compute);
    if (krc) return krc;
    UK_CUDA(cudaEventRecord(pipe->out_ready[j], pipe->compute));
    UK_CUDA(cudaStreamWaitEvent(pipe->d2h, pipe->out_ready[j], 0));
    UK_CUDA(cudaMemcpy2DAsync(h_out + c.begin * a.out_tile_bytes, size_t(h_out_pitch), d_slab,
                              size_t(slab_row), size_t(slab_row), size_t(p.M),
                              cudaMemcpyDeviceToHost, pipe->d2h));
    slab_off += p.M * slab_row;
  }
  // the caller's stream completes when the last slab is on the host
  UK_CUDA(cudaEventRecord(pipe->done, pipe->d2h));
  UK_CUDA(cudaStreamWaitEvent(user, pipe->done, 0));
#undef UK_CUDA
  return IREE_UK_B200_OK;
}

}  // extern "C"
