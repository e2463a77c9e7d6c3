// Internal declarations shared by the translation units of libiree_uk_b200.so.
#ifndef IREE_UK_B200_CSRC_UK_COMMON_H_
#define IREE_UK_B200_CSRC_UK_COMMON_H_

#include <cuda_runtime.h>

#include <atomic>
#include <stddef.h>
#include <stdint.h>

#include "../../include/iree_uk_b200.h"

namespace uk {

// Element types of the path, by width and interpretation.
enum class Elem : int { F32, S32, F16, BF16, S16, S8, U4, S4 };

inline int elem_bits(Elem e) {
  switch (e) {
    case Elem::F32: case Elem::S32: return 32;
    case Elem::F16: case Elem::BF16: case Elem::S16: return 16;
    case Elem::S8: return 8;
    default: return 4;
  }
}

// (lhs, rhs, out) of a mmt4d type id; false when the id is not a mmt4d type.
// Mirrors iree_uk_mmt4d_type (ukernel/mmt4d_internal.h:63-97).
struct Mmt4dTypes {
  Elem lhs, rhs, out;
};
bool mmt4d_types(uint32_t flags, Mmt4dTypes* t);

// Bytes per element of a pack / unpack type id, 0 when invalid
// (ukernel/pack_internal.h:43-59, unpack_internal.h:39-53).
int pack_elem_size(uint32_t flags);
int unpack_elem_size(uint32_t flags);

// Host-side restatements of the reference's *_validate functions. Return IREE_UK_B200_OK
// or IREE_UK_B200_INVALID_ARGUMENT.
int validate_mmt4d(const iree_uk_mmt4d_params_t* p);    // ukernel/mmt4d.c:12-48
int validate_pack(const iree_uk_pack_params_t* p);      // ukernel/pack.c:51-104
int validate_unpack(const iree_uk_unpack_params_t* p);  // ukernel/unpack.c:31-82

// ---- launchers (each enqueues on `stream`, returns a status) -------------------------

int launch_mmt4d_generic(const iree_uk_mmt4d_params_t* p, cudaStream_t stream);
int launch_mmt4d_zero_fill(const iree_uk_mmt4d_params_t* p, cudaStream_t stream);
int launch_mmt4d_gemv_s16u4(const iree_uk_mmt4d_params_t* p, cudaStream_t stream);
bool mmt4d_gemv_s16u4_eligible(const iree_uk_mmt4d_params_t* p);
// Narrowed M0 (1, 2, 4, 8) x N0 = 16 tiles of s8s8s32 / f16f16f32 / bf16bf16f32: weight streaming.
bool mmt4d_narrow_eligible(const iree_uk_mmt4d_params_t* p);
int launch_mmt4d_narrow(const iree_uk_mmt4d_params_t* p, cudaStream_t stream);

// Output of a tensor-core mmt4d written as a row-major rows x cols matrix (the unpack folded
// into the epilogue); p->out_buffer / out_offset / out_stride0 then describe that matrix.
struct RowMajorOut {
  int64_t rows, cols;
};
bool mmt4d_tc_operands_eligible(const iree_uk_mmt4d_params_t* p);
// Tensor-core path. `variant` selects the operand staging layout (see uk_mmt4d_tc.cu).
bool mmt4d_tc_eligible(const iree_uk_mmt4d_params_t* p);
// s16u4s32 1x32x8 with enough rows to fill tensor-core tiles (two byte planes x u8 weights).
bool mmt4d_tc_s16u4_eligible(const iree_uk_mmt4d_params_t* p);
// s16s16s32 16x16x2 (two byte planes of both operands, four 8-bit products per term).
bool mmt4d_tc_s16s16_eligible(const iree_uk_mmt4d_params_t* p);
// s16s8s32 16x16x2 (two byte planes of the LHS against the s8 RHS, two products per term).
bool mmt4d_tc_s16s8_eligible(const iree_uk_mmt4d_params_t* p);
// s8s4s32 16x16xK0 (K0 = 2, 4, 8, 16): nibbles widened to bytes by the pre-pass, then s8s8s32.
bool mmt4d_tc_s8s4_eligible(const iree_uk_mmt4d_params_t* p);
int launch_mmt4d_tc_s8s4(const iree_uk_mmt4d_params_t* p, void* ws, size_t ws_bytes, int variant,
                         cudaStream_t stream);
size_t mmt4d_tc_workspace_size(const iree_uk_mmt4d_params_t* p);
// `peer_out_buffers`: optional device pointers (usually on other GPUs) that stand for
// p->out_buffer in further copies of the output; every tile is stored to all of them too.
// `multicast_out`: alternatively, the NVLink multicast mapping that stands for p->out_buffer
// on every GPU of a group; tiles are then stored once, through multimem.st.
int launch_mmt4d_tc(const iree_uk_mmt4d_params_t* p, void* ws, size_t ws_bytes, int variant,
                    cudaStream_t stream, const void* const* peer_out_buffers = nullptr,
                    int num_peers = 0, const void* multicast_out = nullptr,
                    const void* prepared_rhs = nullptr, const RowMajorOut* row_major_out = nullptr);
// `prepared_rhs`: the RHS already re-tiled by launch_mmt4d_tc_prepare_rhs (weights prepared
// once); the call then re-tiles only the LHS and needs mmt4d_tc_prepared_workspace_size bytes.
size_t mmt4d_tc_prepared_rhs_size(const iree_uk_mmt4d_params_t* p);
size_t mmt4d_tc_prepared_workspace_size(const iree_uk_mmt4d_params_t* p);
int launch_mmt4d_tc_prepare_rhs(const iree_uk_mmt4d_params_t* p, void* prepared, size_t bytes,
                                cudaStream_t stream);
// Row-major matmul on the tensor-core kernels (lhs [M][K], rhs [K][N], out [M][N] 32-bit);
// pitches in bytes, out_stride0 in elements.
size_t matmul_workspace_size(uint32_t flags, int64_t M, int64_t N, int64_t K);
int launch_matmul_rowmajor(uint32_t flags, const char* lhs, int64_t lhs_pitch_b, const char* rhs,
                           int64_t rhs_pitch_b, char* out, int64_t out_stride0, int64_t M, int64_t N,
                           int64_t K, void* ws, size_t ws_bytes, cudaStream_t stream);
// Tensor-core mmt4d without scratch (operands re-tiled on the way into shared memory).
bool mmt4d_tc_sw_eligible(const iree_uk_mmt4d_params_t* p);
int launch_mmt4d_tc_sw(const iree_uk_mmt4d_params_t* p, cudaStream_t stream);
// Process-wide choice for f32f32f32 with 16x16 tiles: 0 = CUDA cores in the reference's
// accumulation order (default), 1 = tensor cores, three tf32 products per term.
int f32_mode();
constexpr int kTcVariantDefault = 0;
constexpr int kTcVariantDirect = 3;  // MN-major, 32-byte swizzle, straight from the operand
constexpr int kTcVariantTwoCta = 5;  // CTA pairs, both operands by TMA from re-tiled scratch
constexpr int kTcVariantOneCta = 6;  // one CTA per tile, both operands by TMA
constexpr int kTcVariantStreamed = 7;  // CTA pairs; the kernel's own workers finish the re-tile
// f16f16f32 / bf16bf16f32 with M0 = N0 = 16 and K0 = 1: served by the tensor cores without scratch.
bool mmt4d_tc_direct_eligible(const iree_uk_mmt4d_params_t* p);

int launch_pack_generic(const iree_uk_pack_params_t* p, cudaStream_t stream);
int launch_unpack_generic(const iree_uk_unpack_params_t* p, cudaStream_t stream);
// Shared-memory staged relayouts; return IREE_UK_B200_UNSUPPORTED when the shape does not
// fit their staging buffer (the caller then uses the generic kernel).
int launch_pack_staged(const iree_uk_pack_params_t* p, cudaStream_t stream);
int launch_unpack_staged(const iree_uk_unpack_params_t* p, cudaStream_t stream);
bool pack_staged_eligible(const iree_uk_pack_params_t* p);
bool unpack_staged_eligible(const iree_uk_unpack_params_t* p);

int launch_interleave_slabs(const void* gathered, void* out, int64_t M, int64_t N,
                            int64_t tile_elems, int elem_size, int world, cudaStream_t stream);

// Per-device status word written by kernels whose bounded waits ran out.
// Returns a device pointer valid on the current device, or nullptr on CUDA failure.
uint32_t* device_status_word();

inline int cuda_status(cudaError_t e) {
  return e == cudaSuccess ? IREE_UK_B200_OK : IREE_UK_B200_CUDA_ERROR;
}

// Optional kernel timing for benchmarks (off by default, see iree_uk_b200_kernel_timing): when
// enabled on a device, launchers that run a pre-pass plus a main kernel record CUDA events
// between them on the launching stream. One ring per device, created on that device; the
// counters are atomics, so concurrent callers lose no slot. A recorded call runs without the
// overlap of its pre-pass and main kernel (the event between them serialises the two), which is
// why only every n-th call is recorded.
struct KernelTiming {
  static constexpr int kRing = 64;  // calls remembered
  std::atomic<bool> enabled{false};
  std::atomic<int> every{1};          // record one call in `every` (the others run unobserved)
  std::atomic<long long> seen{0};     // tensor-core calls since timing was enabled
  cudaEvent_t ev[kRing][3] = {};      // per recorded call: before pre-pass, before main, after main
  std::atomic<long long> calls{0};    // calls recorded since timing was enabled
  // The event triple for this call, or nullptr when the call is not to be recorded.
  cudaEvent_t* next_slot() {
    if (!enabled.load(std::memory_order_relaxed)) return nullptr;
    const long long n = seen.fetch_add(1, std::memory_order_relaxed);
    if (n % every.load(std::memory_order_relaxed)) return nullptr;
    return ev[calls.load(std::memory_order_relaxed) % kRing];
  }
  // Records `e` on `stream`; a failure is cleared so that it cannot be mistaken for a launch
  // error by the caller's own cudaGetLastError().
  static void record(cudaEvent_t e, cudaStream_t stream) {
    if (cudaEventRecord(e, stream) != cudaSuccess) cudaGetLastError();
  }
};
// The timing ring of the current device (nullptr when the device cannot be determined).
KernelTiming* kernel_timing();

// Test hook (iree_uk_b200_testing_starve_producers): true while the producers of the
// tensor-core kernels are told to fill nothing, which makes the bounded waits run out.
bool testing_starve_producers();

// True when the environment variable is set to a non-empty value other than "0".
bool env_flag(const char* name);

// Tuning overrides read from the environment. They exist only in a build made with
// -DIREE_UK_B200_EXPERIMENTS (parameter sweeps); the shipped library always takes `fallback`.
#ifdef IREE_UK_B200_EXPERIMENTS
int debug_int(const char* name, int fallback);
#else
constexpr int debug_int(const char*, int fallback) { return fallback; }
#endif

}  // namespace uk

#endif  // IREE_UK_B200_CSRC_UK_COMMON_H_
