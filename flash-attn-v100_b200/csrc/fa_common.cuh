// Shared declarations of the library's translation units: the C-ABI header,
// error plumbing, and the per-family launch entry points host_api.cu routes to.
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>
#include "../../include/fa_b200.h"
#include "philox.cuh"

namespace fa {

// Thread-local detail string behind fa_b200_last_error().
void set_error(const char* fmt, ...);

#define FA_CUDA_CHECK(expr)                                                        \
    do {                                                                           \
        cudaError_t _e = (expr);                                                   \
        if (_e != cudaSuccess) {                                                   \
            fa::set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e),  \
                          __FILE__, __LINE__);                                     \
            return FA_ECUDA;                                                       \
        }                                                                          \
    } while (0)

// ---- dtype helpers ---------------------------------------------------------
template <typename T> __device__ __forceinline__ float to_f32(T x);
template <> __device__ __forceinline__ float to_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ float to_f32<__half>(__half x) { return __half2float(x); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }

template <typename T> __device__ __forceinline__ T from_f32(float x);
template <> __device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ __half from_f32<__half>(float x) { return __float2half_rn(x); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

static inline size_t dtype_bytes(int dtype) { return dtype == FA_B200_F32 ? 4 : 2; }
static inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// Keys batch entry b attends to: its entry of the optional per-batch count array, clamped to [1, Nk].
__device__ __forceinline__ int kv_len_of(const int32_t* lens, int b, int Nk) {
    if (!lens) return Nk;
    const int l = lens[b];
    return l < 1 ? 1 : (l > Nk ? Nk : l);
}

// Origin of the call's (batch, head) columns in the dropout stream (rng_heads = 0: the call is the whole problem).
static inline DropoutOrigin dropout_origin_of(const fa_b200_params& p) {
    DropoutOrigin o;
    o.b0 = p.rng_batch_offset;
    o.h0 = p.rng_head_offset;
    o.heads = p.rng_heads > 0 ? p.rng_heads : p.H;
    return o;
}

// ---- workspace layout (backward) -------------------------------------------
// [ delta : B*H*nq_pad fp32 | lse*log2(e) : B*H*nq_pad fp32 | ranges : B*Hkv x {max|dO|, max|V|} fp32
//   | row exponents of dO : B*H*nq_pad fp32 | fp16 copies of Q, dO (B*Nq*H*D each) and K (B*Nk*Hkv*D)
//   | dQ sums : B*H*nq_pad*D fp32 ]
// every region starts on a 256-byte boundary.  delta alone serves the CUDA-core family (which
// indexes it unpadded); lse and ranges belong to the tensor-core family; the row exponents and
// the fp16 copies to its bf16 calls (tcgen05.mma wants one format for both operands, see
// sm100_ptx.cuh) unless `inline_conversion` is asked for, which converts the tiles inside the main
// kernels instead and needs no copies; the dQ sums to the one-kernel backward.
// nq_pad = Nq rounded up to 128.
struct BwdWorkspace {
    size_t delta_off, delta_bytes;
    size_t lse2_off, lse2_bytes;
    size_t rng_off, rng_bytes;
    size_t erow_off, erow_bytes;
    size_t q16_off, q16_bytes;
    size_t do16_off, do16_bytes;
    size_t k16_off, k16_bytes;
    size_t dq_off, dq_bytes;
    size_t total;
};
BwdWorkspace bwd_workspace_layout(const fa_b200_params& p, int variant, bool inline_conversion = false);

// ---- kernel families ---------------------------------------------------------
// CUDA-core tiles (simt_kernels.cu)
int simt_fwd(const fa_b200_params& p);
int simt_bwd(const fa_b200_params& p, const BwdWorkspace& ws);
bool simt_supports(const fa_b200_params& p);

// TMA + tcgen05 (fwd_sm100.cu, bwd_sm100.cu)
int sm100_fwd(const fa_b200_params& p);
int sm100_bwd(const fa_b200_params& p, const BwdWorkspace& ws);
bool sm100_supports(const fa_b200_params& p, bool backward, const char** why);
// fp32 forward on the tensor cores (fwd_tf32_sm100.cu): TF32 products taken three times
int sm100_tf32_fwd(const fa_b200_params& p);
bool sm100_tf32_fwd_supports(const fa_b200_params& p, const char** why);
// Whether the one-kernel backward (dQ summed with global additions) covers a call the family supports.
bool sm100_bwd_fused_supported(const fa_b200_params& p);

// Number of SMs of a device (cached per device; 0 on failure).
int sm_count(int device);

int launch_dropout_mask(uint64_t seed, uint64_t offset, float p, int B, int H, int Nq, int Nk,
                        uint8_t* out, cudaStream_t stream);
// The call's keep bits for the tensor-core kernels (simt_kernels.cu): mq query-major, mk key-major, either may be null.
size_t dropout_bits_bytes(const fa_b200_params& p);
int launch_dropout_bits(const fa_b200_params& p, void* mq, void* mk);

}  // namespace fa
