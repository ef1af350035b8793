// Attention forward for fp32 inputs on the sm_100a tensor cores: tcgen05.mma kind::tf32 with every
// product taken three times (hi*hi + lo*hi + hi*lo), accumulators in tensor memory.
//
// The reference's Triton forward lets fp32 inputs take TF32 tensor-core products with fp32
// accumulation (tl.dot(..., allow_tf32=True), kernels/forward_kernel.py:167,216).  One TF32 product
// keeps 11 significant bits of each operand and misses the fp32 tolerance of this build (1e-5) by
// more than an order of magnitude, so each fp32 operand x is split into
//     hi = x with its low 13 mantissa bits cleared   (exactly a TF32 number)
//     lo = x - hi                                     (exact in fp32; TF32 keeps its leading 11 bits)
// and  a*b  is taken as  hi_a*hi_b + lo_a*hi_b + hi_a*lo_b  (what is dropped is below 2^-21 of the
// product), all three accumulated by the tensor core into one fp32 accumulator.  This holds for both
// contractions: S = Q K^T with Q and K split in shared memory, and O += P V with P split by the
// softmax threads as they write it to tensor memory and V split in shared memory.
//
// One CTA per 128-row query tile of one (batch, head); key/value blocks of 64 rows, two stages.
//   warps 0-3   one thread per query row: operand splits, softmax (exact fp32, log2 domain), epilogue
//   warp 4      one elected thread: TMA loads and MMA issue
// TMEM columns: S [0,64)  P_hi [64,128)  P_lo [128,192)  O [192,192+D).
// Head dimension 64; no dropout and no bias (those calls, other head dimensions and the fp32 backward
// are served by the CUDA-core tiles).  Every mbarrier wait is bounded (sm100_ptx.cuh).
#include "fa_common.cuh"
#include "sm100_ptx.cuh"
#include "tma_host.cuh"

namespace fa {
namespace {

using namespace ptx;

constexpr int kM = 128;            // query rows per CTA
constexpr int kN = 64;             // keys per block
constexpr int kD = 64;             // head dimension
constexpr int kStages = 2;
constexpr int kQBox = kM * 128;    // one TMA box of Q: 128 rows x 32 fp32
constexpr int kKBox = kN * 128;    // one TMA box of K or V: 64 rows x 32 fp32
constexpr int kQTile = (kD / 32) * kQBox;      // 32 KB
constexpr int kKTile = (kD / 32) * kKBox;      // 16 KB
constexpr int kThreads = 160;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

// barrier slots
enum { kBarQ = 0, kBarQSplit = 1, kBarKV = 2 /*[2]*/, kBarKVSplit = 4 /*[2]*/, kBarKVFree = 6 /*[2]*/,
       kBarS = 8, kBarP = 9, kBarO = 10, kNumBars = 11 };
// Q hi | Q lo | per stage: K hi, K lo, V hi, V lo | barriers | tmem slot, wait control
constexpr int kSmemBytes = 2 * kQTile + kStages * 4 * kKTile + kNumBars * 8 + 64 + 1024;

struct Tf32Args {
    float* o; int64_t o_sb, o_sn, o_sh;
    float* lse;
    int32_t* status;
    const int32_t* kv_len;
    int B, Nq, Nk, H, Hkv;
    int causal, shift;
    int wait_limit_ms;
    float scale_log2;
};

// tcgen05.mma kind::tf32 instruction descriptor: fp32 accumulate (bit 4), A and B format TF32 (2) at
// bits 7-9 and 10-12, B major at bit 16 (0 = K-major, 1 = MN-major), N >> 3 at 17, M >> 4 at 24.
__host__ __device__ constexpr uint32_t make_idesc_tf32(int M, int N, bool b_mn_major) {
    return (1u << 4) | (2u << 7) | (2u << 10) | ((b_mn_major ? 1u : 0u) << 16) |
           ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}
__device__ __forceinline__ void mma_ss_tf32(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ void mma_ts_tf32(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(acc) : "memory");
}

// x -> (hi, lo) for `bytes` of fp32 at `hi` (in place) and `lo`; thread t of 128 takes 16-byte pieces
// t, t + 128, ...  Element-wise, so the tiles' swizzle is irrelevant (lo gets the same arrangement).
__device__ __forceinline__ void split_tile(uint8_t* hi, uint8_t* lo, int bytes, int t) {
    uint4* ph = reinterpret_cast<uint4*>(hi) + t;
    uint4* pl = reinterpret_cast<uint4*>(lo) + t;
#pragma unroll 4
    for (int i = 0; i < bytes / (16 * 128); ++i) {
        const uint4 x = ph[i * 128];
        uint4 h, l;
        h.x = x.x & 0xFFFFE000u; l.x = __float_as_uint(__uint_as_float(x.x) - __uint_as_float(h.x));
        h.y = x.y & 0xFFFFE000u; l.y = __float_as_uint(__uint_as_float(x.y) - __uint_as_float(h.y));
        h.z = x.z & 0xFFFFE000u; l.z = __float_as_uint(__uint_as_float(x.z) - __uint_as_float(h.z));
        h.w = x.w & 0xFFFFE000u; l.w = __float_as_uint(__uint_as_float(x.w) - __uint_as_float(h.w));
        ph[i * 128] = h;
        pl[i * 128] = l;
    }
}

__global__ void __launch_bounds__(kThreads, 1)
fwd_tf32_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                const __grid_constant__ CUtensorMap map_v, const Tf32Args a) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* sQh = smem;
    uint8_t* sQl = sQh + kQTile;
    uint8_t* sKV = sQl + kQTile;                 // stage s: K hi, K lo, V hi, V lo (kKTile each)
    uint64_t* bars = (uint64_t*)(sKV + kStages * 4 * kKTile);
    uint32_t* tmem_slot = (uint32_t*)(bars + kNumBars);
    volatile uint32_t* abort_flag = (volatile uint32_t*)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // Blocks are dispatched in linear order: walk the tiles slowest and the (batch, head) columns fastest,
    // heavy tiles (under a causal mask the last ones) first, so that the longest blocks of ALL columns start
    // first and the short ones fill the end (B2 N1024 H12: 192 blocks of 1 to 8 units on 148 SMs).
    const int n_cols = (int)(gridDim.y * gridDim.z);
    const int lin = (int)(blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z));
    const int slow = lin / n_cols, col = lin - slow * n_cols;
    const int tile = a.causal ? (int)gridDim.x - 1 - slow : slow;
    const int h = col % (int)gridDim.y, b = col / (int)gridDim.y;
    const int hk = h / (a.H / a.Hkv);
    const int nk = kv_len_of(a.kv_len, b, a.Nk);
    int kv_end = nk;
    if (a.causal && tile * kM + kM + a.shift < kv_end) kv_end = tile * kM + kM + a.shift;
    const int nblk = (kv_end + kN - 1) / kN;

    if (threadIdx.x == 0) {
        for (int i = 0; i < kNumBars; ++i) {
            const bool workers = (i == kBarQSplit || i == kBarKVSplit || i == kBarKVSplit + 1 || i == kBarP);
            mbar_init(&bars[i], workers ? 4u : 1u);       // one arrival per worker warp
        }
        wait_control_init(abort_flag, a.wait_limit_ms);
        fence_mbar_init();
    }
    if (warp == 4) {
        tmem_alloc(tmem_slot, 256);
        tmem_relinquish();
        if (lane == 0) { prefetch_tensormap(&map_q); prefetch_tensormap(&map_k); prefetch_tensormap(&map_v); }
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;
    const uint32_t tS = tmem, tPh = tmem + 64u, tPl = tmem + 128u, tO = tmem + 192u;

    if (warp == 4) {
        // ------------------------------------------------------------ TMA + MMA (one thread)
        if (elect_one()) {
            constexpr uint32_t idesc_s = make_idesc_tf32(kM, kN, false);      // S: B = K block, K-major
            constexpr uint32_t idesc_pv = make_idesc_tf32(kM, kD, true);      // O: B = V block, MN-major
            const uint32_t sQh_u = smem_u32(sQh), sQl_u = smem_u32(sQl), sKV_u = smem_u32(sKV);
            const uint64_t dk_major = make_smem_desc_sw128(0, 0, 1024);
            // V is MN-major (N = head dim): a 32-bit MN-major operand has one arrangement, the 128-byte
            // swizzle in 32-byte pieces (TMA delivers it so): 4-row groups of 512 bytes along K
            const uint64_t dmn_major = make_smem_desc(0, kKBox, 512, 1u);
            auto load_kv = [&](int j) {
                const int s = j % kStages;
                uint8_t* base = sKV + s * 4 * kKTile;
                mbar_expect_tx(&bars[kBarKV + s], 2 * kKTile);
#pragma unroll
                for (int bx = 0; bx < kD / 32; ++bx) {
                    tma_load_4d(base + bx * kKBox, &map_k, &bars[kBarKV + s], bx * 32, hk, j * kN, b);
                    tma_load_4d(base + 2 * kKTile + bx * kKBox, &map_v, &bars[kBarKV + s], bx * 32, hk, j * kN, b);
                }
            };
            // S (+)= A[tile] * B[tile]^T, both K-major: D / 8 K-steps of 8 fp32 (32 bytes); a box holds 32
            auto issue_s = [&](uint32_t a_u, uint32_t b_u, bool acc) {
                const uint64_t a0 = dk_major + (uint64_t)(a_u >> 4), b0 = dk_major + (uint64_t)(b_u >> 4);
#pragma unroll
                for (int kk = 0; kk < kD / 8; ++kk) {
                    const uint32_t ao = ((uint32_t)(kk >> 2) * kQBox + (uint32_t)(kk & 3) * 32u) >> 4;
                    const uint32_t bo = ((uint32_t)(kk >> 2) * kKBox + (uint32_t)(kk & 3) * 32u) >> 4;
                    mma_ss_tf32(tS, a0 + ao, b0 + bo, idesc_s, (acc || kk > 0) ? 1u : 0u);
                }
            };
            // O (+)= P[TMEM] * V[tile], V MN-major: kN / 8 K-steps of 8 keys (8 rows of 128 bytes)
            auto issue_pv = [&](uint32_t p_tmem, uint32_t v_u, bool acc) {
                const uint64_t b0 = dmn_major + (uint64_t)(v_u >> 4);
#pragma unroll
                for (int kk = 0; kk < kN / 8; ++kk)
                    mma_ts_tf32(tO, p_tmem + (uint32_t)kk * 8u, b0 + (uint64_t)((kk * 1024) >> 4), idesc_pv,
                                (acc || kk > 0) ? 1u : 0u);
            };
            bool ok = true;
            if (nblk > 0) {
                mbar_expect_tx(&bars[kBarQ], kQTile);
#pragma unroll
                for (int bx = 0; bx < kD / 32; ++bx)
                    tma_load_4d(sQh + bx * kQBox, &map_q, &bars[kBarQ], bx * 32, h, tile * kM, b);
                load_kv(0);
                if (nblk > 1) load_kv(1);
                ok = mbar_wait(&bars[kBarQSplit], 0u, abort_flag);
            }
            for (int j = 0; j < nblk && ok; ++j) {
                const int s = j % kStages;
                const uint32_t ph = (uint32_t)(j / kStages) & 1u;
                const uint32_t base = sKV_u + (uint32_t)(s * 4 * kKTile);
                ok = mbar_wait(&bars[kBarKVSplit + s], ph, abort_flag);
                if (!ok) break;
                tc_fence_after_sync();
                issue_s(sQh_u, base, false);                 // Q_hi K_hi
                issue_s(sQl_u, base, true);                  // Q_lo K_hi
                issue_s(sQh_u, base + kKTile, true);         // Q_hi K_lo
                mma_commit(&bars[kBarS]);
                ok = mbar_wait(&bars[kBarP], (uint32_t)j & 1u, abort_flag);
                if (!ok) break;
                tc_fence_after_sync();
                issue_pv(tPh, base + 2 * kKTile, j > 0);     // P_hi V_hi
                issue_pv(tPl, base + 2 * kKTile, true);      // P_lo V_hi
                issue_pv(tPh, base + 3 * kKTile, true);      // P_hi V_lo
                mma_commit(&bars[kBarKVFree + s]);           // the stage's tiles have been read
                mma_commit(&bars[kBarO]);
                if (j + kStages < nblk) {
                    ok = mbar_wait(&bars[kBarKVFree + s], ph, abort_flag);
                    if (!ok) break;
                    load_kv(j + kStages);
                }
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------ splits, softmax, epilogue
        const int t = threadIdx.x;                        // 0..127: query row of the tile = TMEM lane
        const uint32_t lane_off = (uint32_t)(warp * 32) << 16;
        const int i = tile * kM + t;                      // global query row
        float m = -INFINITY, l = 0.f;
        bool ok = true;
        if (nblk > 0) {
            ok = mbar_wait(&bars[kBarQ], 0u, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (ok) {
                split_tile(sQh, sQl, kQTile, t);
                fence_proxy_async_smem();
                mbar_arrive_warp(&bars[kBarQSplit]);
            }
        }
        for (int j = 0; j < nblk && ok; ++j) {
            const int s = j % kStages;
            const uint32_t ph = (uint32_t)(j / kStages) & 1u;
            uint8_t* base = sKV + s * 4 * kKTile;
            ok = mbar_wait(&bars[kBarKV + s], ph, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            split_tile(base, base + kKTile, kKTile, t);                     // K
            split_tile(base + 2 * kKTile, base + 3 * kKTile, kKTile, t);    // V
            fence_proxy_async_smem();
            mbar_arrive_warp(&bars[kBarKVSplit + s]);

            ok = mbar_wait(&bars[kBarS], (uint32_t)j & 1u, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after_sync();
            uint32_t sr[2][32];
            tmem_ld_32x32(tS + lane_off, sr[0]);
            tmem_ld_32x32(tS + lane_off + 32u, sr[1]);
            tmem_wait_ld();
            // my row sees the block's first `seen` columns: keys below the count, at most i + shift
            const int col0 = j * kN;
            int seen = nk - col0;
            if (a.causal && i + a.shift + 1 - col0 < seen) seen = i + a.shift + 1 - col0;
            float mx = -INFINITY;
#pragma unroll
            for (int c = 0; c < kN; ++c) {
                float x = __uint_as_float(sr[c >> 5][c & 31]) * a.scale_log2;
                if (c >= seen) x = -INFINITY;
                sr[c >> 5][c & 31] = __float_as_uint(x);
                mx = fmaxf(mx, x);
            }
            const float m_new = fmaxf(m, mx);
            // a row that has seen no key yet (possible only beyond Nq) keeps m = -inf: its P are exp2(-inf - (-inf));
            // use 0 as the reference there so that they come out as 0
            const float m_ref = (m_new == -INFINITY) ? 0.f : m_new;
            // the accumulator is rescaled by the whole warp or not at all (tensor-memory accesses are
            // warp-collective): a row whose maximum stays gets alpha = 1
            if (__any_sync(0xffffffffu, m_new > m)) {
                const float alpha = exp2f(m - m_ref);              // 0 on the first block
                l *= alpha;
                if (j > 0) {
                    // O(j-1) is complete: its MMAs were committed to the O barrier before S(j) was issued
                    ok = mbar_wait(&bars[kBarO], (uint32_t)(j - 1) & 1u, abort_flag);
                    ok = __all_sync(0xffffffffu, ok);
                    if (ok) {
                        tc_fence_after_sync();
#pragma unroll
                        for (int c0 = 0; c0 < kD; c0 += 32) {
                            uint32_t orr[32];
                            tmem_ld_32x32(tO + lane_off + c0, orr);
                            tmem_wait_ld();
#pragma unroll
                            for (int c = 0; c < 32; ++c) orr[c] = __float_as_uint(__uint_as_float(orr[c]) * alpha);
                            tmem_st_32x32(tO + lane_off + c0, orr);
                        }
                    }
                }
                m = m_new;
            }
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            float sum = 0.f;
            uint32_t plo[2][32];
#pragma unroll
            for (int c = 0; c < kN; ++c) {
                const float p = exp2f(__uint_as_float(sr[c >> 5][c & 31]) - m_ref);
                sum += p;
                const uint32_t hi = __float_as_uint(p) & 0xFFFFE000u;
                sr[c >> 5][c & 31] = hi;
                plo[c >> 5][c & 31] = __float_as_uint(p - __uint_as_float(hi));
            }
            l += sum;
            tmem_st_32x32(tPh + lane_off, sr[0]);
            tmem_st_32x32(tPh + lane_off + 32u, sr[1]);
            tmem_st_32x32(tPl + lane_off, plo[0]);
            tmem_st_32x32(tPl + lane_off + 32u, plo[1]);
            tmem_wait_st();
            tc_fence_before_sync();
            mbar_arrive_warp(&bars[kBarP]);
        }
        // ---- epilogue
        if (nblk > 0 && ok) ok = mbar_wait(&bars[kBarO], (uint32_t)(nblk - 1) & 1u, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (ok && nblk > 0) {
            tc_fence_after_sync();
            const float inv = 1.f / l;
            float* orow = a.o + (int64_t)b * a.o_sb + (int64_t)i * a.o_sn + (int64_t)h * a.o_sh;
#pragma unroll
            for (int c0 = 0; c0 < kD; c0 += 32) {
                uint32_t orr[32];
                tmem_ld_32x32(tO + lane_off + c0, orr);
                tmem_wait_ld();
                if (i < a.Nq) {
#pragma unroll
                    for (int g = 0; g < 8; ++g)
                        *reinterpret_cast<float4*>(orow + c0 + g * 4) =
                            make_float4(__uint_as_float(orr[g * 4]) * inv, __uint_as_float(orr[g * 4 + 1]) * inv,
                                        __uint_as_float(orr[g * 4 + 2]) * inv, __uint_as_float(orr[g * 4 + 3]) * inv);
                }
            }
            if (i < a.Nq) a.lse[((int64_t)b * a.H + h) * a.Nq + i] = kLn2 * (m + log2f(l));
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == 4) tmem_dealloc(tmem, 256);
    if (threadIdx.x == 0 && *abort_flag) report_status(a.status, 5);
}

bool fp32_tensor_ok(const fa_b200_tensor& t, int64_t B, int64_t N, int64_t H) {
    if (((uintptr_t)t.ptr & 15u) != 0) return false;
    if (H > 1 && (t.stride_h % 4) != 0) return false;
    if (N > 1 && (t.stride_n % 4) != 0) return false;
    if (B > 1 && (t.stride_b % 4) != 0) return false;
    return true;
}

}  // namespace

// Which fp32 forward calls the TF32 kernel covers.
bool sm100_tf32_fwd_supports(const fa_b200_params& p, const char** why) {
    if (p.dtype != FA_B200_F32) { *why = "dtype must be fp32"; return false; }
    if (p.D != kD) { *why = "head_dim must be 64"; return false; }
    if (p.bias.ptr) { *why = "an additive bias is served by the CUDA-core kernels"; return false; }
    if (dropout_threshold(p.dropout_p) != 0u) { *why = "dropout is served by the CUDA-core kernels"; return false; }
    if (p.o_lo.ptr) { *why = "fp32 output has no rounding residual"; return false; }
    if (!(p.scale > 0.f) || !(p.scale < 1e30f)) { *why = "scale must be positive and finite"; return false; }
    if (p.B > 65535 || p.H > 65535) { *why = "batch and heads must be below 65536"; return false; }
    if (!fp32_tensor_ok(p.q, p.B, p.Nq, p.H) || !fp32_tensor_ok(p.k, p.B, p.Nk, p.Hkv) ||
        !fp32_tensor_ok(p.v, p.B, p.Nk, p.Hkv) || !fp32_tensor_ok(p.o, p.B, p.Nq, p.H)) {
        *why = "tensors must be 16-byte aligned with strides that are multiples of 4 elements";
        return false;
    }
    *why = "";
    return true;
}

int sm100_tf32_fwd(const fa_b200_params& p) {
    CUtensorMap mq, mk, mv;
    int r;
    const CUtensorMapDataType dt = CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
    if ((r = cached_tmap_bnhd(&mq, p.q.ptr, dt, 4, p.B, p.Nq, p.H, kD, p.q.stride_b, p.q.stride_n, p.q.stride_h, kM, 32, true)) ||
        (r = cached_tmap_bnhd(&mk, p.k.ptr, dt, 4, p.B, p.Nk, p.Hkv, kD, p.k.stride_b, p.k.stride_n, p.k.stride_h, kN, 32, true)) ||
        (r = cached_tmap_bnhd(&mv, p.v.ptr, dt, 4, p.B, p.Nk, p.Hkv, kD, p.v.stride_b, p.v.stride_n, p.v.stride_h, kN, 32, 2))) {
        set_error("cuTensorMapEncodeTiled failed (%d)", r);
        return FA_ECUDA;
    }
    Tf32Args a;
    a.o = (float*)p.o.ptr; a.o_sb = p.o.stride_b; a.o_sn = p.o.stride_n; a.o_sh = p.o.stride_h;
    a.lse = p.lse; a.status = p.status_word; a.kv_len = p.kv_lengths;
    a.B = p.B; a.Nq = p.Nq; a.Nk = p.Nk; a.H = p.H; a.Hkv = p.Hkv;
    a.causal = p.causal; a.shift = p.causal ? p.causal_shift : 0;
    a.wait_limit_ms = p.wait_limit_ms;
    a.scale_log2 = p.scale * kLog2e;
    {
        static std::mutex mu;
        static uint64_t done = 0;
        FA_CUDA_CHECK(set_smem_limit_once(fwd_tf32_kernel, kSmemBytes, p.device, &done, &mu));
    }
    const dim3 grid((p.Nq + kM - 1) / kM, p.H, p.B);
    fwd_tf32_kernel<<<grid, kThreads, kSmemBytes, (cudaStream_t)p.stream>>>(mq, mk, mv, a);
    FA_CUDA_CHECK(cudaGetLastError());
    return FA_OK;
}

}  // namespace fa
