// Running combination of per-block partial results, for sequence-parallel
// attention: every rank holds a slice of the sequence, key/value blocks travel
// around a ring, and each (query slice, key block) pair is one ordinary forward
// or backward call whose result has to be folded into a running total.
//
//   outputs    acc <- acc * e^(lse_acc - lse') + part * e^(lse_part - lse'),
//              lse' = log(e^lse_acc + e^lse_part)          (lse_acc != nullptr)
//   gradients  acc <- acc + part                           (lse_acc == nullptr)
//
// The totals stay in fp32 between steps; the step that is known to be the last
// one for a tensor also writes the total in the tensors' own dtype.  The
// reference's sequence-parallel path is a stub that falls back to splitting
// heads (interface.py:437-450), so there is no reference kernel behind this.
//
// HBM-bound streaming kernel: 8 elements per thread (two 16-byte fp32 accesses,
// one 16-byte access of a 16-bit partial), grid = a multiple of the SM count.
#include "fa_common.cuh"

namespace fa {
namespace {

struct CombineArgs {
    float* acc;
    float* lse_acc;
    const void* part;
    const float* lse_part;
    void* out;
    int64_t part_sb, part_sn, part_sh;
    int64_t out_sb, out_sn, out_sh;
    int64_t acc_sb;             // batch stride of acc (elements); rows of one batch entry are dense
    int64_t lse_sb, lse_sh;     // batch and head strides of lse_acc (lse_part is dense)
    int N, H, D;
    int64_t n_chunks;           // B * N * H * 2^cshift
    int cshift;                 // 2^cshift >= D / 8
    int first;
};

template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&x)[8]);

template <>
__device__ __forceinline__ void load8<float>(const float* p, float (&x)[8]) {
    const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
    x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w; x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
}
template <>
__device__ __forceinline__ void load8<__half>(const __half* p, float (&x)[8]) {
    const uint4 r = *reinterpret_cast<const uint4*>(p);
    const __half2* h = reinterpret_cast<const __half2*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 f = __half22float2(h[i]); x[2 * i] = f.x; x[2 * i + 1] = f.y; }
}
template <>
__device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float (&x)[8]) {
    const uint4 r = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); x[2 * i] = f.x; x[2 * i + 1] = f.y; }
}

template <typename T>
__device__ __forceinline__ void store8(T* p, const float (&x)[8]);

template <>
__device__ __forceinline__ void store8<float>(float* p, const float (&x)[8]) {
    reinterpret_cast<float4*>(p)[0] = make_float4(x[0], x[1], x[2], x[3]);
    reinterpret_cast<float4*>(p)[1] = make_float4(x[4], x[5], x[6], x[7]);
}
template <>
__device__ __forceinline__ void store8<__half>(__half* p, const float (&x)[8]) {
    uint4 r;
    __half2* h = reinterpret_cast<__half2*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(x[2 * i], x[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = r;
}
template <>
__device__ __forceinline__ void store8<__nv_bfloat16>(__nv_bfloat16* p, const float (&x)[8]) {
    uint4 r;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(x[2 * i], x[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = r;
}

// MERGE: weights from the two log-sum-exps; otherwise a plain sum.  Idx: the type the element index is
// taken apart in (32-bit whenever the tensor allows it: 64-bit divisions are emulated and would
// make this streaming kernel ALU-bound).
template <typename T, bool MERGE, typename Idx>
__global__ void __launch_bounds__(256) combine_kernel(const CombineArgs a) {
    // A (b, n, h) row of D / 8 chunks takes 2^cshift consecutive threads (the surplus ones idle), so a
    // row never straddles a warp: its threads read the old log-sum-exp with one warp-wide load, on
    // which the one store of the new value depends.
    const int cpr = a.D >> 3;
    const Idx total = (Idx)a.n_chunks, step = (Idx)(gridDim.x * blockDim.x);
    for (Idx idx = (Idx)(blockIdx.x * blockDim.x + threadIdx.x); idx < total; idx += step) {
        const Idx row_i = idx >> a.cshift;                      // (b * N + n) * H + h
        const int c = (int)(idx & (Idx)((1 << a.cshift) - 1));
        if (c >= cpr) continue;
        const Idx bn = row_i / (Idx)a.H;
        const int h = (int)(row_i - bn * (Idx)a.H);
        const Idx b_i = bn / (Idx)a.N;
        const int n = (int)(bn - b_i * (Idx)a.N);
        const int64_t b = (int64_t)b_i;
        float wa = a.first ? 0.f : 1.f, wp = a.part ? 1.f : 0.f;
        if (MERGE) {
            const int64_t li = b * a.lse_sb + h * a.lse_sh + n;
            const float lp = a.part ? a.lse_part[(b * a.H + h) * a.N + n] : -INFINITY;
            const float la = a.first ? -INFINITY : a.lse_acc[li];
            const float m = fmaxf(la, lp);
            float ln = -INFINITY;
            wa = wp = 0.f;
            if (m > -INFINITY) {                                // otherwise no key has been seen yet
                wa = __expf(la - m);
                wp = __expf(lp - m);
                const float s = wa + wp;
                ln = m + __logf(s);
                wa = __fdividef(wa, s);
                wp = __fdividef(wp, s);
            }
            // every lane of the row has read the old log-sum-exp above before one of them replaces it
            // (independent thread scheduling gives no such order by itself)
            __syncwarp(__activemask());
            if (c == 0) a.lse_acc[li] = ln;
        }
        float x[8], y[8];
        float* accp = a.acc + b * a.acc_sb + ((int64_t)n * a.H + h) * a.D + c * 8;
        if (a.first) {
#pragma unroll
            for (int i = 0; i < 8; ++i) x[i] = 0.f;
        } else {
            load8<float>(accp, x);
        }
        if (a.part) {
            load8<T>(reinterpret_cast<const T*>(a.part) + b * a.part_sb + n * a.part_sn + h * a.part_sh + c * 8, y);
#pragma unroll
            for (int i = 0; i < 8; ++i) x[i] = x[i] * wa + y[i] * wp;
            store8<float>(accp, x);
        }
        if (a.out) store8<T>(reinterpret_cast<T*>(a.out) + b * a.out_sb + n * a.out_sn + h * a.out_sh + c * 8, x);
    }
}

template <typename T>
int launch(const CombineArgs& a, bool merge, int device, cudaStream_t stream) {
    const int sms = sm_count(device);
    if (sms <= 0) { set_error("cannot read the SM count of device %d", device); return FA_ECUDA; }
    int64_t blocks = (a.n_chunks + 255) / 256;
    const int64_t cap = (int64_t)sms * 8;                       // 8 resident CTAs of 256 threads per SM
    if (blocks > cap) blocks = cap;
    // idx + one grid stride must not wrap
    const bool small = a.n_chunks + blocks * 256 < (int64_t)0x7fffffff;
    if (merge) {
        if (small) combine_kernel<T, true, uint32_t><<<(unsigned)blocks, 256, 0, stream>>>(a);
        else       combine_kernel<T, true, int64_t><<<(unsigned)blocks, 256, 0, stream>>>(a);
    } else {
        if (small) combine_kernel<T, false, uint32_t><<<(unsigned)blocks, 256, 0, stream>>>(a);
        else       combine_kernel<T, false, int64_t><<<(unsigned)blocks, 256, 0, stream>>>(a);
    }
    FA_CUDA_CHECK(cudaGetLastError());
    return FA_OK;
}

}  // namespace
}  // namespace fa

using namespace fa;

extern "C" int fa_b200_combine(const fa_b200_combine_params* p) {
    if (!p) { set_error("params is null"); return FA_EINVAL; }
    if (p->struct_bytes != sizeof(fa_b200_combine_params)) {
        set_error("struct_bytes %zu does not match this library's fa_b200_combine_params (%zu bytes)",
                  p->struct_bytes, sizeof(fa_b200_combine_params));
        return FA_EINVAL;
    }
    if (p->B < 0 || p->N < 0 || p->H < 0 || p->D <= 0) { set_error("negative size"); return FA_EINVAL; }
    if (p->D > 256) { set_error("D=%d: the combination kernel takes rows of at most 256 elements", p->D); return FA_EUNSUPPORTED; }
    if (p->D % 8 != 0) { set_error("D=%d: the combination kernel moves 8 elements per thread", p->D); return FA_EUNSUPPORTED; }
    if (p->dtype != FA_B200_F16 && p->dtype != FA_B200_BF16 && p->dtype != FA_B200_F32) {
        set_error("bad dtype %d", p->dtype);
        return FA_EINVAL;
    }
    const int64_t rows = (int64_t)p->B * p->N * p->H;
    if (rows == 0) return FA_OK;
    if (!p->acc) { set_error("acc is null"); return FA_EINVAL; }
    if (!p->part.ptr && !p->out.ptr) { set_error("neither a partial nor an output: nothing to do"); return FA_EINVAL; }
    if (!p->part.ptr && p->first) { set_error("first step without a partial"); return FA_EINVAL; }
    const bool merge = p->lse_acc != nullptr;
    if (merge && p->part.ptr && !p->lse_part) { set_error("lse_acc without lse_part"); return FA_EINVAL; }
    const size_t esz = p->dtype == FA_B200_F32 ? 4 : 2;
    auto aligned = [&](const fa_b200_tensor& t) {
        return ((uintptr_t)t.ptr % 16 == 0) && (t.stride_b * esz % 16 == 0) && (t.stride_n * esz % 16 == 0) &&
               (t.stride_h * esz % 16 == 0);
    };
    if (p->acc_stride_b % 4 != 0 || p->acc_stride_b < 0 || p->lse_stride_b < 0 || p->lse_stride_h < 0) {
        set_error("acc_stride_b must be a non-negative multiple of 4 elements, lse strides non-negative");
        return FA_EALIGN;
    }
    if ((uintptr_t)p->acc % 16 != 0 || (p->part.ptr && !aligned(p->part)) || (p->out.ptr && !aligned(p->out))) {
        set_error("acc, part and out must be 16-byte aligned with strides that are multiples of 16 bytes");
        return FA_EALIGN;
    }
    CombineArgs a;
    a.acc = p->acc; a.lse_acc = p->lse_acc; a.part = p->part.ptr; a.lse_part = p->lse_part; a.out = p->out.ptr;
    a.part_sb = p->part.stride_b; a.part_sn = p->part.stride_n; a.part_sh = p->part.stride_h;
    a.out_sb = p->out.stride_b; a.out_sn = p->out.stride_n; a.out_sh = p->out.stride_h;
    a.N = p->N; a.H = p->H; a.D = p->D;
    a.acc_sb = p->acc_stride_b ? p->acc_stride_b : (int64_t)p->N * p->H * p->D;
    a.lse_sb = p->lse_stride_b ? p->lse_stride_b : (int64_t)p->H * p->N;
    a.lse_sh = p->lse_stride_h ? p->lse_stride_h : (int64_t)p->N;
    a.cshift = 0;
    while ((1 << a.cshift) < p->D / 8) ++a.cshift;
    a.n_chunks = rows << a.cshift;
    a.first = p->first ? 1 : 0;
    int prev = -1;
    if (cudaGetDevice(&prev) != cudaSuccess) { set_error("cudaGetDevice failed"); return FA_ECUDA; }
    if (prev != p->device && cudaSetDevice(p->device) != cudaSuccess) {
        set_error("cudaSetDevice(%d) failed", p->device);
        return FA_ECUDA;
    }
    cudaStream_t stream = (cudaStream_t)p->stream;
    int rc;
    if (p->dtype == FA_B200_F16) rc = launch<__half>(a, merge, p->device, stream);
    else if (p->dtype == FA_B200_BF16) rc = launch<__nv_bfloat16>(a, merge, p->device, stream);
    else rc = launch<float>(a, merge, p->device, stream);
    if (prev != p->device) cudaSetDevice(prev);
    return rc;
}
