// Attention backward for sm_100a: TMA -> shared memory -> tcgen05.mma with
// accumulators in tensor memory, warp-specialised.
//
// Replaces the reference's Triton backward kernel
// (kernels/backward_kernel.py:17-205) and its launcher (:208-318).
//
// Three launches:
//   1. preprocess  -delta = -rowsum(dO o O) and -lse*log2(e), both fp32, written
//                  to the workspace in rows padded to whole 128-row tiles
//                  (padding: delta = 0, -lse = -inf, so padded queries get P = 0)
//   2. MODE 0      one CTA per 128-row key tile (stationary K, V), streams the
//                  query tiles: writes dK and dV
//   3. MODE 1      one CTA per 128-row query tile (stationary Q, dO), streams
//                  the key tiles: writes dQ
// Every output element is owned by one CTA and accumulated in a fixed order, so
// results are bit-reproducible (the reference accumulates dQ across CTAs with
// an unordered read-modify-write, kernels/backward_kernel.py:179-194).
//
// D = 64 has a faster route (MODE 2) unless the two-pass variant is asked for:
// the key-stationary kernel also forms the step's dQ tile, dS K_j, from the
// dS^T tile its threads leave in shared memory, and adds it to an fp32 buffer in
// global memory (red.global.add.v4.f32, order across CTAs not fixed); S and dP
// are then computed once instead of twice.  Launches: memset of the buffer +
// preprocess, MODE 2, and a conversion of the sums to dQ.  At D = 128 tensor
// memory has no columns left for the dQ tile and the additions cost more than
// the second kernel's recomputation, so that size keeps the two passes.
//
// Both modes run the same pipeline on a stationary pair (X, Y) and a streamed
// pair (U, W):
//                         MODE 0 (dK, dV)          MODE 1 (dQ)
//   X, Y                  K_j, V_j                 Q_i, dO_i
//   U, W                  Q_i, dO_i                K_j, V_j
//   T1 = X U^T            S^T                      S
//   T2 = Y W^T            dP^T                     dP
//   phase A (T1 -> P)     P^T = exp2(S^T c - lse)  P = exp2(S c - lse)
//   phase B (T2 -> dS)    dS^T = P^T o (dP^T o Z - delta)
//   ACC2 += P  W          dV += (P o Z)^T dO       (not computed)
//   ACC1 += dS U          dK += dS^T Q             dQ += dS K
// T1/T2 are SS MMAs (both operands K-major in shared memory); the accumulating
// MMAs take P / dS from TMEM (written over T1 / T2 by the threads that read
// them) and U / W from the same shared-memory tiles read MN-major.
//
//   warps 0-15       four elementwise warpgroups; a thread owns one TMEM lane (row)
//                    and warpgroup g owns columns [32g, 32g+32) of T1/T2
//   warp 16          MMA issuer; order  T1(0) T2(0) | ACC2(i) T1(i+1) ACC1(i) T2(i+1) ...  (MODE 0, 2)
//                                       T1(0) T2(0) | T1(i+1) T2(i+1) ACC1(i) ...          (MODE 1)
//   warp 17          TMA producer: U and W tiles into rings of their own (U is read again by the
//                    step's last MMA, so it gets three stages where shared memory allows and its
//                    next load overlaps a whole step; W gets two), and in the key-stationary
//                    kernels the step's -lse / -delta rows into a two-slot ring
//   warps 18-19      bf16 inputs: convert the streamed tiles to fp16 in place as they land (all MMAs run
//                    f16 x f16, with P and dS rounded to fp16; see "number formats" below); else idle
//
// TMEM columns: T1 [0,128)  T2 [128,256)  ACC1 [256,256+D)  ACC2 [384,384+D).
// MODE 1 has no ACC2 and never writes P back (only dS is an MMA operand there): S has the one buffer
// T1, free again once the threads hold S(i) in registers, and dP / dS alternate between T2 and
// [384,512), so that S(i+1) and dP(i+1) are both computed while the threads work on step i.
// MODE 2 (D = 64) puts the dQ tile at [448,512).
// Every mbarrier wait is bounded; see sm100_ptx.cuh.
#include "fa_common.cuh"
#include "sm100_ptx.cuh"
#include "tma_host.cuh"
#include "tile_config.cuh"
#include <type_traits>

namespace fa {
namespace {

using namespace ptx;

constexpr int kTile = 128;
constexpr int kBoxBytes = 128 * 128;
constexpr int kNWG = tile::kBwdWarpgroups;   // elementwise warpgroups per CTA (each owns 128 / kNWG columns)
constexpr int kExtraThreads = 128;       // MMA warp + TMA warp + two idle warps: registers are granted per
                                         // four warps, so dropping the idle pair would free none
constexpr float kLog2e = 1.4426950408889634f;

// Shared-memory plan of one kernel instance.  The streamed tiles U and W have rings of their own:
// U (Q_i in the key-stationary kernels, K_j in MODE 1) is read by the first MMA of its step and again
// by the last one, a step and a half later, so two stages leave the TMA load of the next tile no
// time at all (it can only start when the last reader has finished and is needed at once); W is
// done within one step.  D = 128 has room for three U stages and two W stages, except that the
// key-stationary dropout instance needs 4 KB for its masks and stays at two and two.
// DROP: 0 no dropout; 1 keep bits drawn by the kernel's own threads; 2 loaded from the call's bit buffer.
template <int D, int MODE, int DROP>
struct BwdCfg {
    static constexpr int kNBox = D / 64;
    static constexpr int kTileBytes = kNBox * kBoxBytes;
    static constexpr bool kFused = (MODE == 2);
    static constexpr bool kMasks = DROP == 1 && MODE != 1;       // masks are built in shared memory when keys are rows
    static constexpr int kUStages = tile::bwd_u_stages(D, kMasks);
    static constexpr int kWStages = tile::bwd_w_stages(D);
    static constexpr int kMaskBytes = 2 * 128 * 8 * 2;          // two buffers of 128 x 8 uint16 keep masks
    static constexpr int kXYFull = 0;
    static constexpr int kUFull = 1;                             // [kUStages]
    static constexpr int kUEmpty = kUFull + kUStages;            // [kUStages]
    static constexpr int kWFull = kUEmpty + kUStages;            // [kWStages]
    static constexpr int kWEmpty = kWFull + kWStages;            // [kWStages]
    static constexpr int kT1Full = kWEmpty + kWStages;           // [2]: one per S buffer (MODE 0 uses the first)
    static constexpr int kT2Full = kT1Full + 2;
    static constexpr int kPReady = kT2Full + 1;                  // one arrival per elementwise warp
    static constexpr int kDsReady = kPReady + 1;                 // one arrival per elementwise warp
    static constexpr int kAccDone = kDsReady + 1;
    static constexpr int kMask = kAccDone + 1;                   // one arrival per elementwise warp
    static constexpr int kEpi = kMask + 1;                       // one arrival per elementwise warp
    static constexpr int kDqFull = kEpi + 1;                     // fused kernel: dQ tile of the step complete
    static constexpr int kDqRead = kDqFull + 1;                  // ... and read out (one arrival per warp)
    static constexpr int kPHalf = kDqRead + 1;                   // key-stationary: first half of each P^T slice stored
    static constexpr int kDsHalf = kPHalf + 1;                   // first half of each dS slice stored
    static constexpr int kVFull = kDsHalf + 1;                   // [2] key-stationary: -lse, -delta rows of a step landed
    static constexpr int kVEmpty = kVFull + 2;                   // [2] ... and read (one arrival per elementwise warp)
    // bf16 inputs: tiles converted to fp16 in place (arrivals: one per converting warp)
    static constexpr int kXYConv = kVEmpty + 2;                  // stationary tiles (elementwise warps)
    static constexpr int kUConv = kXYConv + 1;                   // [kUStages] streamed U (the two spare warps)
    static constexpr int kWConv = kUConv + kUStages;             // [kWStages] streamed W, key-stationary kernels only
    static constexpr int kNumBars = kWConv + kWStages;
    static constexpr int kVecBytes = (MODE != 1) ? 2 * 1024 : 0; // two slots of lse[128] | delta[128]
    static constexpr int kDsBytes = 128 * 128 * 2;               // fused kernel: dS^T tile for the dQ MMA
    // bytes used from the 1024-aligned base: X, Y, U ring, W ring, [dS], [vectors], barriers, TMEM slot + flag, [masks]
    static constexpr int kUsedBytes = (2 + kUStages + kWStages) * kTileBytes + (kFused ? kDsBytes : 0) + kVecBytes +
                                      kNumBars * 8 + 64 + (kMasks ? kMaskBytes : 0);
    static constexpr int kMaxSmem = 232448;                      // 227 KB: the most one CTA can ask for
    static_assert(128 * kNWG + 128 == 32 * tile::kBwdWarps, "thread count and table disagree");
    static_assert(kUsedBytes <= kMaxSmem, "shared-memory plan does not fit");
    // what the launch asks for: room to align the base when it fits (the kernel checks what it got)
    static constexpr int kSmemBytes = kUsedBytes + 1024 <= kMaxSmem ? kUsedBytes + 1024 : kMaxSmem;
};

struct BwdArgs {
    const float* lse2;     // [B*H][nq_pad]  kPShift - lse * log2(e), -inf in the padding
    const float* delta;    // [B*H][nq_pad]  -delta, 0 in the padding
    const float* ranges;   // [B*Hkv][2]     max |dO| over the column's query heads, max |V|
    const float* erow;     // [B*H][nq_pad]  row exponents e_i of the fp16 dO copy (row form only)
    float* dq_acc;         // fused kernel: fp32 dQ sums, [B*H][nq_pad/128] tiles of [D/4][128 rows][4]
    const int32_t* kv_len; // optional per-batch key counts
    int32_t* status;
    int B, Nq, Nk, H, Hkv, nq_pad;
    int wait_limit_ms;             // limit of one mbarrier wait (0: the default)
    int cols_per_group;            // CTA order: (batch, head) columns per group, see cta_work()
    int causal;
    int shift;                     // key j is visible to query i iff j <= i + shift
    float scale, scale_log2;
    uint32_t drop_thr;
    float inv_keep;
    PhiloxKey key;
    DropoutOrigin rng;
    // DROP = 2, the call's keep bits as dropout_bits_kernel lays them out:
    const uint4* bits_q;           // [(b*H + h) * ceil128(Nk)/128 + key tile][nq_pad]: 128 keys of one query row
    const uint32_t* bits_k;        // [((b*H + h) * nq_pad/128 + query tile) * 4 + g][nk_pad]: 32 queries of one key row
    int nk_pad;
};

__device__ __forceinline__ void bulk_load_1d(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(gsrc)), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}

// ---- number formats of the two operands the threads hand to the MMAs -----------------------------
// P and dS are written to tensor memory as fp16 whatever the input dtype (with bf16 they would carry
// a 2^-9 rounding into dV, dK and dQ at full size; see sm100_ptx.cuh), so both are scaled into
// fp16's range by powers of two that the epilogue takes out again:
//   P'  = P * 2^kPShift                      P <= 1, so P' <= 2^14 and P down to 2^-28 keeps 11 bits
//   dS' = P (dP o Z - delta) * 2^g           g from a bound: |dP o Z - delta| <= 2 D max|dO| max|V| / (1-p)
// and, for bf16 inputs, dO is normalised while it is converted to fp16: dO' = dO * 2^-eO, max|dO'| < 2^15,
// so gradients of any magnitude (bf16 training runs with dO ~ 1e-8) use fp16's range.  max|dO| and max|V|
// are taken per (batch, K/V head) column by the preprocess launch, so a column's result does not depend
// on which other columns the call holds.
constexpr float kPShift = 14.0f;

struct BwdScales {
    float tt_mul;     // dP (as the MMA delivers it) * tt_mul
    float nd_mul;     // the staged -delta vector * nd_mul
    float l_add;      // added to the staged lse vector (key-stationary kernels)
    float acc1_mul;   // dK or dQ  = ACC1 * acc1_mul  (scale * 2^-g)
    float acc2_mul;   // dV        = ACC2 * acc2_mul
    float do_mul;     // inline conversion: dO' = dO * do_mul
};
// smallest k with m < 2^k (0 for m == 0; NaN and infinity count as the largest finite exponent)
__host__ __device__ __forceinline__ int log2_bound_bits(uint32_t bits) {
    bits &= 0x7FFFFFFFu;
    if (bits == 0u) return 0;
    int e = (int)(bits >> 23);
    if (e == 0) return -126;
    if (e > 254) e = 254;
    return e - 127 + 1;
}
__device__ __forceinline__ int log2_bound(float m) { return log2_bound_bits(__float_as_uint(m)); }
__device__ __forceinline__ float pow2i(int e) {
    e = e < -126 ? -126 : (e > 127 ? 127 : e);
    return __uint_as_float((uint32_t)(e + 127) << 23);
}
// How dO reaches the key-stationary kernels' MMAs, which decides where its normalisation sits:
//   kDoAsIs     fp16 inputs: dO is used as it is
//   kDoInline   bf16, converted tile by tile inside the kernel: one factor 2^-e_col for the whole column
//   kDoRowCopy  bf16, converted once by the preprocess launch into an fp16 copy, every row by its own
//               2^-e_i (the column's maximum is not known while the copy is written); the staged vectors
//               hold  lse' = kPShift - lse*log2(e) + e_i  and  -delta * 2^-e_i,  and P carries 2^(e_i - e_col)
// With e_col = (bound of the column's max |dO|) - 15 the constants below are the same in the last two
// forms except for l_add and nd_mul.  The query-stationary kernel multiplies the bf16 dO itself
// (kDoAsIs arithmetic; it undoes e_i in its per-row scalars when the vectors are in the row form).
enum DoForm { kDoAsIs = 0, kDoInline = 1, kDoRowCopy = 2 };
__device__ __forceinline__ BwdScales make_scales(const float* rng, int D, float inv_keep, float scale, DoForm form) {
    const int k_do = log2_bound(rng[0]), k_v = log2_bound(rng[1]);
    const int e_col = form == kDoAsIs ? 0 : k_do - 15;
    const int g = 15 - (k_do + k_v + (D > 64 ? 8 : 7) + log2_bound(inv_keep));
    BwdScales sc;
    sc.tt_mul = pow2i(g - (int)kPShift + e_col);
    sc.nd_mul = pow2i(g - (int)kPShift + (form == kDoRowCopy ? e_col : 0));
    sc.l_add = form == kDoRowCopy ? (float)(-e_col) : 0.f;
    sc.acc1_mul = scale * pow2i(-g);
    sc.acc2_mul = inv_keep * pow2i(e_col - (int)kPShift);
    sc.do_mul = pow2i(-e_col);
    return sc;
}

// Which (tile, head, batch) a CTA works on.  The grid is (tiles, heads, batch) and CTAs start in the
// order of their linear index.  Under a causal mask tiles cost between 1 and `tiles` steps, so the
// order decides how evenly the SMs finish: the (batch, head) columns are taken in groups of
// `cols_per_group`, and within a group all columns' most expensive tile comes first, then the next
// one, ... (longest first).  A group is sized so that its Q, K, V and dO stay in L2 while its CTAs
// run; the cheap tiles that end one group fill the SMs beside the expensive ones that start the next.
struct CtaWork { int tile_rank, head, b; };
__device__ __forceinline__ CtaWork cta_work(int cols_per_group) {
    const int X = (int)gridDim.x, Y = (int)gridDim.y, cols = Y * (int)gridDim.z;
    const int L = (int)blockIdx.x + X * ((int)blockIdx.y + Y * (int)blockIdx.z);
    const int G = cols_per_group < 1 ? 1 : cols_per_group;
    const int grp = L / (G * X), r = L - grp * (G * X);
    const int gcols = (cols - grp * G) < G ? (cols - grp * G) : G;
    const int col = grp * G + r % gcols;
    CtaWork w;
    w.tile_rank = r / gcols;
    w.head = col % Y;
    w.b = col / Y;
    return w;
}

// MODE 0: dK, dV (key-stationary).  MODE 1: dQ (query-stationary).
// INLINE (bf16 inputs only): the streamed tiles arrive as bf16 and the two spare warps convert them;
// otherwise bf16 calls stream the fp16 copies the preprocess launch (Q, dO) and the dK/dV kernel (K:
// map_aux, a by-product of its stationary tile) have written to the workspace.
template <int D, bool BF16, int MODE, int NWG, int DROP, bool INLINE>
__global__ void __launch_bounds__(128 * NWG + kExtraThreads, 1)
bwd_sm100_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_y,
                 const __grid_constant__ CUtensorMap map_u, const __grid_constant__ CUtensorMap map_w,
                 const __grid_constant__ CUtensorMap map_out1, const __grid_constant__ CUtensorMap map_out2,
                 const __grid_constant__ CUtensorMap map_aux, const BwdArgs a) {
    using Cfg = BwdCfg<D, MODE, DROP>;
    constexpr bool KS = (MODE != 1);        // key-stationary: K, V stay, query tiles stream
    constexpr bool FUSED = (MODE == 2);     // key-stationary and dQ too
    constexpr bool CONV = BF16;             // every MMA runs f16 x f16: bf16 tiles are converted
    constexpr bool STREAM_CONV = CONV && INLINE;             // ... the streamed ones by the spare warps
    constexpr bool XY_CONV = CONV && (KS || INLINE);         // ... the stationary ones by the elementwise warps
    constexpr bool ROWFORM = CONV && !INLINE;                // staged vectors are in the row form (see DoForm)
    constexpr bool K_COPY = ROWFORM && MODE == 0;            // this kernel writes the fp16 copy of K
    static_assert(BF16 || !INLINE, "inline conversion is a bf16 variant");
    constexpr int UST = Cfg::kUStages, WST = Cfg::kWStages;
    constexpr int TILE = Cfg::kTileBytes;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* sX = smem;
    uint8_t* sY = sX + TILE;
    uint8_t* sU = sY + TILE;                        // U ring
    uint8_t* sW = sU + UST * TILE;                  // W ring
    uint8_t* sDs = sW + WST * TILE;                 // fused kernel only
    float* sVec = (float*)(sDs + (FUSED ? Cfg::kDsBytes : 0));      // key-stationary only: 2 x (lse[128] | delta[128])
    uint64_t* bars = (uint64_t*)((uint8_t*)sVec + Cfg::kVecBytes);
    uint32_t* tmem_slot = (uint32_t*)(bars + Cfg::kNumBars);
    volatile uint32_t* abort_flag = (volatile uint32_t*)(tmem_slot + 1);
    uint16_t* sMask = (uint16_t*)((uint8_t*)bars + Cfg::kNumBars * 8 + 64);    // present with dropout only
    {
        // the launch may have had no room for a full kilobyte of alignment slack
        uint32_t dyn;
        asm volatile("mov.u32 %0, %%dynamic_smem_size;" : "=r"(dyn));
        if ((uint32_t)(smem - smem_raw) + (uint32_t)Cfg::kUsedBytes > dyn) {
            if (threadIdx.x == 0) report_status(a.status, 8);
            return;
        }
    }

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const CtaWork cw = cta_work(a.cols_per_group);
    const int b = cw.b;
    const int group = a.H / a.Hkv;
    const int nq_tiles = (a.Nq + kTile - 1) / kTile;

    // iteration space (uniform over the CTA)
    const int nk = kv_len_of(a.kv_len, b, a.Nk);    // keys this batch entry attends to
    int tile, head_x, it0, n_per_head, n_iter;
    if (KS) {
        tile = cw.tile_rank;                        // key tile: the first one sees the most query tiles
        head_x = cw.head;                           // kv head
        // first query tile that sees this key tile: query i sees key j iff j <= i + shift
        it0 = a.causal ? (tile * kTile > a.shift ? (tile * kTile - a.shift) / kTile : 0) : 0;
        n_per_head = nq_tiles > it0 ? nq_tiles - it0 : 0;
        if (tile * kTile >= nk) n_per_head = 0;     // a tile of padding keys: dK = dV = 0
        n_iter = n_per_head * group;
    } else {
        tile = a.causal ? (int)gridDim.x - 1 - cw.tile_rank : cw.tile_rank;     // query tile, heavy first
        head_x = cw.head;                           // query head
        it0 = 0;
        int kv_end = nk;
        if (a.causal && tile * kTile + kTile + a.shift < kv_end) kv_end = tile * kTile + kTile + a.shift;
        n_per_head = (kv_end + kTile - 1) / kTile;
        n_iter = n_per_head;
    }
    const int head_kv = (KS) ? head_x : head_x / group;
    // Key-stationary kernels: query tile of step `it`.  The fused kernel without a causal mask starts
    // each key tile's walk at a different query tile, so that the CTAs of one head, which run at
    // the same time, add to different dQ tiles (under a causal mask the walks are staggered already).
    const int rot = (FUSED && !a.causal && n_per_head > 0) ? tile % n_per_head : 0;
    // qi = index of the step within its query head (each role keeps qi and the head count as
    // running counters: a division per step and warp is a visible share of the issue slots)
    auto q_tile_of = [&](int qi) {
        int t = qi + rot;
        if (t >= n_per_head) t -= n_per_head;
        return it0 + t;
    };

    if (threadIdx.x == 0) {
        for (int i = 0; i < Cfg::kNumBars; ++i) {
            const bool wide = (i == Cfg::kPReady || i == Cfg::kDsReady || i == Cfg::kMask || i == Cfg::kEpi ||
                               i == Cfg::kDqRead || i == Cfg::kPHalf || i == Cfg::kDsHalf ||
                               i == Cfg::kVEmpty || i == Cfg::kVEmpty + 1 || i == Cfg::kXYConv);
            const bool conv2 = i >= Cfg::kUConv;          // the two converting warps
            mbar_init(&bars[i], wide ? 4u * NWG : (conv2 ? 2u : 1u));    // one arrival per elementwise warp
        }
        wait_control_init(abort_flag, a.wait_limit_ms);
        fence_mbar_init();
    }
    constexpr int kMmaWarp = 4 * NWG, kTmaWarp = 4 * NWG + 1;
    constexpr int CPT = kTile / NWG;                    // columns of T1/T2 one elementwise thread owns
    // The dQ kernel reads nothing the dK/dV kernel writes: it may take the SMs this grid's last wave
    // leaves idle (it is launched serialized behind this grid, and waits for it only before it ends).
    if (MODE == 0) grid_launch_dependents();
    if (warp == kMmaWarp) {
        tmem_alloc(tmem_slot, 512);
        tmem_relinquish();
    }
    if (warp == kTmaWarp && lane == 0) {
        prefetch_tensormap(&map_x); prefetch_tensormap(&map_y);
        prefetch_tensormap(&map_u); prefetch_tensormap(&map_w);
        prefetch_tensormap(&map_out1);
        if (KS) prefetch_tensormap(&map_out2);
        if (K_COPY) prefetch_tensormap(&map_aux);
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;
    const uint32_t tT1 = tmem, tT2 = tmem + 128u, tAcc1 = tmem + 256u, tAcc2 = tmem + 384u;
    // fused kernel: the per-step dQ tile has columns of its own when D = 64 and shares T2's when D = 128
    constexpr bool kDqAliasesT2 = (D > 64);
    const uint32_t tDq = kDqAliasesT2 ? tT2 : tmem + 448u;
    const BwdScales sc = make_scales(a.ranges + 2 * ((int64_t)b * a.Hkv + head_kv), D, a.inv_keep, a.scale,
                                     !(CONV && KS) ? kDoAsIs : (INLINE ? kDoInline : kDoRowCopy));

    // Registers: without dropout the launch allocation of 96 per thread lets no role spill, and moving
    // registers from the MMA / TMA warps to the elementwise ones (104 / 64, 104 / 40) made one side or the
    // other spill and measured the same or slower.  The dK/dV kernel's dropout instances do spill in the
    // elementwise loop at 96 (28 local loads and 24 stores per step and warp, 8 % of the kernel's
    // instructions under ncu): they take 104 and leave 64 to the other warpgroup (1.272 -> 1.216 ms at
    // B32 H16 N2048 D64; the one-kernel backward got slower with the same split, 1.439 -> 1.466, and keeps 96).
    constexpr bool kMoveRegs = DROP != 0 && MODE == 0 && !INLINE;
    // The pool is what the CTA was launched with (96 per thread): a split that asks for more makes
    // setmaxnreg.inc wait for ever (112 / 40 did: 62464 > 61440).
    constexpr int kRegsElementwiseMoved = 104, kRegsOtherMoved = 64, kRegsLaunch = 96;
    static_assert(128 * NWG * kRegsElementwiseMoved + kExtraThreads * kRegsOtherMoved <= (128 * NWG + kExtraThreads) * kRegsLaunch,
                  "register split exceeds the launch allocation");
    if (warp >= kMmaWarp) {
      if constexpr (kMoveRegs) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsOtherMoved));
      if (warp == kTmaWarp) {
        // ---------------------------------------------------------------- TMA producer
        if (elect_one()) {
            int u_issued = 0, w_issued = 0, v_issued = 0;
            bool ok = true;
            if (n_iter > 0) {
                mbar_expect_tx(&bars[Cfg::kXYFull], 2 * TILE);
#pragma unroll
                for (int bx = 0; bx < Cfg::kNBox; ++bx) {
                    tma_load_4d(sX + bx * kBoxBytes, &map_x, &bars[Cfg::kXYFull], bx * 64, head_x, tile * kTile, b);
                    tma_load_4d(sY + bx * kBoxBytes, &map_y, &bars[Cfg::kXYFull], bx * 64, head_x, tile * kTile, b);
                }
            }
            int qi = 0, hg = 0;
            int us = 0, ws = 0;                      // ring slots of this step
            uint32_t uph = 0, wph = 0;               // how often each ring has wrapped (parity)
            for (int it = 0; it < n_iter; ++it) {
                int head_u, row_u;
                if (KS) { head_u = head_x * group + hg; row_u = q_tile_of(qi) * kTile; }
                else    { head_u = head_kv; row_u = it * kTile; }
                ok = mbar_wait(&bars[Cfg::kUEmpty + us], (uph & 1u) ^ 1u, abort_flag);
                if (!ok) break;
                mbar_expect_tx(&bars[Cfg::kUFull + us], TILE);
#pragma unroll
                for (int bx = 0; bx < Cfg::kNBox; ++bx)
                    tma_load_4d(sU + us * TILE + bx * kBoxBytes, &map_u, &bars[Cfg::kUFull + us], bx * 64, head_u, row_u, b);
                ++u_issued;
                ok = mbar_wait(&bars[Cfg::kWEmpty + ws], (wph & 1u) ^ 1u, abort_flag);
                if (!ok) break;
                mbar_expect_tx(&bars[Cfg::kWFull + ws], TILE);
#pragma unroll
                for (int bx = 0; bx < Cfg::kNBox; ++bx)
                    tma_load_4d(sW + ws * TILE + bx * kBoxBytes, &map_w, &bars[Cfg::kWFull + ws], bx * 64, head_u, row_u, b);
                ++w_issued;
                if (KS) {
                    // the step's -lse*log2(e) and -delta rows: a two-slot ring of their own
                    const int vs = it & 1;
                    ok = mbar_wait(&bars[Cfg::kVEmpty + vs], ((uint32_t)(it >> 1) & 1u) ^ 1u, abort_flag);
                    if (!ok) break;
                    const int64_t off = ((int64_t)b * a.H + head_u) * a.nq_pad + row_u;
                    mbar_expect_tx(&bars[Cfg::kVFull + vs], 1024);
                    bulk_load_1d(sVec + vs * 256, a.lse2 + off, 512, &bars[Cfg::kVFull + vs]);
                    bulk_load_1d(sVec + vs * 256 + 128, a.delta + off, 512, &bars[Cfg::kVFull + vs]);
                    ++v_issued;
                }
                if (++us == UST) { us = 0; ++uph; }
                if (++ws == WST) { ws = 0; ++wph; }
                if (++qi == n_per_head) { qi = 0; ++hg; }
            }
            if (!ok) {
                // unwinding: let copies already issued land before shared memory is given up
                for (int st = 0; st < UST; ++st) {
                    const int nf = (u_issued + UST - 1 - st) / UST;
                    for (int spin = 0; spin < 4096 && nf > 0 &&
                         !mbar_try_wait(&bars[Cfg::kUFull + st], (uint32_t)(nf - 1) & 1u); ++spin) {}
                }
                for (int st = 0; st < WST; ++st) {
                    const int nf = (w_issued + WST - 1 - st) / WST;
                    for (int spin = 0; spin < 4096 && nf > 0 &&
                         !mbar_try_wait(&bars[Cfg::kWFull + st], (uint32_t)(nf - 1) & 1u); ++spin) {}
                }
                for (int st = 0; st < 2; ++st) {
                    const int nf = (v_issued + 1 - st) / 2;
                    for (int spin = 0; spin < 4096 && nf > 0 &&
                         !mbar_try_wait(&bars[Cfg::kVFull + st], (uint32_t)(nf - 1) & 1u); ++spin) {}
                }
                for (int spin = 0; spin < 4096 && n_iter > 0 && !mbar_try_wait(&bars[Cfg::kXYFull], 0u); ++spin) {}
            }
        }
        __syncwarp();
      } else if (warp == kMmaWarp) {
        // ---------------------------------------------------------------- MMA issuer
        if (elect_one() && n_iter > 0) {
            // operand formats: converted tiles, P and dS are fp16; the query-stationary kernel's dP keeps
            // its two bf16 tiles (dO_i, V_j) as they are
            constexpr bool T1_BF16 = BF16 && !CONV, T2_BF16 = BF16 && !(CONV && KS);
            constexpr uint32_t idesc_t1 = make_idesc_f16(T1_BF16, T1_BF16, kTile, kTile, false, false);
            constexpr uint32_t idesc_t2 = make_idesc_f16(T2_BF16, T2_BF16, kTile, kTile, false, false);
            constexpr uint32_t idesc_acc = make_idesc_f16(false, false, kTile, D, false, true);
            constexpr int kUReady = STREAM_CONV ? Cfg::kUConv : Cfg::kUFull;
            constexpr int kWReady = (STREAM_CONV && KS) ? Cfg::kWConv : Cfg::kWFull;
            constexpr int kXYReady = XY_CONV ? Cfg::kXYConv : Cfg::kXYFull;
            const uint32_t sX_u = smem_u32(sX), sY_u = smem_u32(sY), sU_u = smem_u32(sU), sW_u = smem_u32(sW);

            // Descriptors differ only in the 16-byte-granular start address held in their low
            // bits: build the two kinds once and add offsets in the issue loops, which keeps the
            // single issuing thread's instruction count per MMA small.
            const uint64_t dk_major = make_smem_desc_sw128(0, 0, 1024);            // K-major operand
            const uint64_t dmn_major = make_smem_desc_sw128(0, kBoxBytes, 1024);   // MN-major operand
            auto issue_t = [&](uint32_t d_tmem, uint32_t stat_u, uint32_t strm_u, uint32_t idesc_t) {
                const uint64_t a0 = dk_major + (uint64_t)(stat_u >> 4), b0 = dk_major + (uint64_t)(strm_u >> 4);
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const uint32_t off = ((uint32_t)(kk >> 2) * kBoxBytes + (uint32_t)(kk & 3) * 32u) >> 4;
                    mma_ss_f16(d_tmem, a0 + off, b0 + off, idesc_t, kk > 0);
                }
            };
            // acc (+)= A[TMEM] * B[smem tile, MN-major].  A holds 16-bit pairs: the thread group that owns
            // columns [g*CPT, (g+1)*CPT) of T wrote its CPT values packed into columns [g*CPT, g*CPT + CPT/2).
            auto issue_acc = [&](uint32_t d_tmem, uint32_t a_tmem, uint32_t strm_u, bool acc) {
                const uint64_t b0 = dmn_major + (uint64_t)(strm_u >> 4);
#pragma unroll
                for (int kk = 0; kk < kTile / 16; ++kk) {
                    const uint32_t a_col = (uint32_t)((16 * kk) / CPT) * CPT + (uint32_t)((16 * kk) % CPT) / 2u;
                    mma_ts_f16(d_tmem, a_tmem + a_col, b0 + (uint64_t)((kk * 2048) >> 4), idesc_acc,
                               (acc || kk > 0) ? 1u : 0u);
                }
            };
            // the same product restricted to the first (hf = 0) or second 16 columns of every
            // warpgroup's slice: K-steps kk = hf, hf + 2, hf + 4, hf + 6
            auto issue_acc_half = [&](uint32_t d_tmem, uint32_t a_tmem, uint32_t strm_u, bool acc, int hf) {
                static_assert(CPT == 32, "one K-step of 16 per half slice");
                const uint64_t b0 = dmn_major + (uint64_t)(strm_u >> 4);
#pragma unroll
                for (int g = 0; g < kTile / 32; ++g) {
                    const int kk = 2 * g + hf;
                    const uint32_t a_col = (uint32_t)g * CPT + (uint32_t)hf * 8u;
                    mma_ts_f16(d_tmem, a_tmem + a_col, b0 + (uint64_t)((kk * 2048) >> 4), idesc_acc,
                               (acc || hf > 0 || g > 0) ? 1u : 0u);
                }
            };

            // fused kernel: the step's dQ tile (fresh accumulation) from two shared-memory operands
            constexpr uint32_t idesc_dq = make_idesc_f16(false, false, kTile, D, true, true);
            const uint32_t sDs_u = smem_u32(sDs);
            auto issue_dq = [&]() {
                const uint64_t a0 = dmn_major + (uint64_t)(sDs_u >> 4), b0 = dmn_major + (uint64_t)(sX_u >> 4);
#pragma unroll
                for (int kk = 0; kk < kTile / 16; ++kk)
                    mma_ss_f16(tDq, a0 + (uint64_t)((kk * 2048) >> 4), b0 + (uint64_t)((kk * 2048) >> 4), idesc_dq,
                               kk > 0);
            };

            bool ok = mbar_wait(&bars[kXYReady], 0u, abort_flag);
            if (ok) ok = mbar_wait(&bars[kUReady + 0], 0u, abort_flag);
            if (ok) ok = mbar_wait(&bars[kWReady + 0], 0u, abort_flag);
            if (ok) {
                tc_fence_after_sync();
                issue_t(tT1, sX_u, sU_u, idesc_t1);
                mma_commit(&bars[Cfg::kT1Full]);
                issue_t(tT2, sY_u, sW_u, idesc_t2);
                mma_commit(&bars[Cfg::kT2Full]);
                if (!KS) mma_commit(&bars[Cfg::kWEmpty + 0]);        // MODE 1: V_j is read by dP(j) only
            }
            int us = 0, ws = 0;                      // ring slots of this step's U and W
            uint32_t uph = 0, wph = 0;               // wrap counts (parity of the slots' phases)
            for (int it = 0; it < n_iter && ok; ++it) {
                int nus = us + 1, nws = ws + 1;      // slots of the next step
                uint32_t nuph = uph, nwph = wph;
                if (nus == UST) { nus = 0; ++nuph; }
                if (nws == WST) { nws = 0; ++nwph; }
                const uint32_t cur_u = sU_u + us * TILE, nxt_u = sU_u + nus * TILE;
                const uint32_t cur_w = sW_u + ws * TILE, nxt_w = sW_u + nws * TILE;
                const bool more = it + 1 < n_iter;
                if (more) { ok = mbar_wait(&bars[kUReady + nus], nuph & 1u, abort_flag); if (!ok) break; }
                if (KS) {
                    ok = mbar_wait(&bars[Cfg::kPHalf], (uint32_t)it & 1u, abort_flag);
                    if (!ok) break;
                    tc_fence_after_sync();
                    issue_acc_half(tAcc2, tT1, cur_w, it > 0, 0);                // dV += (P o Z)^T dO, first halves
                    ok = mbar_wait(&bars[Cfg::kPReady], (uint32_t)it & 1u, abort_flag);
                    if (!ok) break;
                    tc_fence_after_sync();
                    issue_acc_half(tAcc2, tT1, cur_w, it > 0, 1);
                    mma_commit(&bars[Cfg::kWEmpty + ws]);                        // dO_i: dP^T(i) earlier, dV(i) last
                    if (more) { issue_t(tT1, sX_u, nxt_u, idesc_t1); mma_commit(&bars[Cfg::kT1Full]); }
                } else if (more) {
                    // dQ needs no second accumulator, and P never goes back to tensor memory here: S has one
                    // buffer, free again as soon as the threads hold S(it) in registers, and dP / dS have
                    // two (T2 and the columns a second accumulator would take).  S(it+1) and dP(it+1) are
                    // both issued before this thread waits for dS(it), so the threads find their next
                    // inputs ready; with one dP buffer, dP(it+1) could only follow dQ(it), and
                    // dS -> dQ -> dP -> dS was the loop that set the step time.
                    ok = mbar_wait(&bars[Cfg::kPReady], (uint32_t)it & 1u, abort_flag);     // S(it) is in registers
                    if (!ok) break;
                    tc_fence_after_sync();
                    issue_t(tT1, sX_u, nxt_u, idesc_t1);
                    mma_commit(&bars[Cfg::kT1Full]);
                    ok = mbar_wait(&bars[kWReady + nws], nwph & 1u, abort_flag);
                    if (!ok) break;
                    tc_fence_after_sync();
                    // the buffer of step it+1 held dS(it-1), which dQ(it-1) read: issued before, in order
                    issue_t(((it + 1) & 1) ? tAcc2 : tT2, sY_u, nxt_w, idesc_t2);
                    mma_commit(&bars[((it + 1) & 1) ? Cfg::kT1Full + 1 : Cfg::kT2Full]);
                    mma_commit(&bars[Cfg::kWEmpty + nws]);
                }
                // query-stationary: a barrier pair per dP / dS buffer (phase = uses of that buffer), which
                // the threads cannot lap: dS(it+2) needs dP(it+2), issued after these waits
                const int b_half = (!KS && (it & 1)) ? Cfg::kPHalf : Cfg::kDsHalf;
                const int b_ready = (!KS && (it & 1)) ? Cfg::kDqRead : Cfg::kDsReady;
                const uint32_t ds_par = KS ? ((uint32_t)it & 1u) : ((uint32_t)(it >> 1) & 1u);
                const uint32_t tDs = (!KS && (it & 1)) ? tAcc2 : tT2;
                ok = mbar_wait(&bars[b_half], ds_par, abort_flag);
                if (!ok) break;
                tc_fence_after_sync();
                issue_acc_half(tAcc1, tDs, cur_u, it > 0, 0);                    // dK += dS^T Q  /  dQ += dS K
                ok = mbar_wait(&bars[b_ready], ds_par, abort_flag);
                if (!ok) break;
                tc_fence_after_sync();
                issue_acc_half(tAcc1, tDs, cur_u, it > 0, 1);
                mma_commit(&bars[Cfg::kUEmpty + us]);                            // last reader of U(it)
                if (FUSED) {
                    // dQ tile of this step = dS K_j: A is the dS^T tile the threads left in shared memory,
                    // read MN-major (M = queries), B is the stationary K tile read MN-major (N = D)
                    if (!kDqAliasesT2 && it > 0) {
                        // own columns: only the previous tile's read-out has to precede (issuing
                        // dP^T(it+1) ahead of this MMA measured slower)
                        ok = mbar_wait(&bars[Cfg::kDqRead], (uint32_t)(it - 1) & 1u, abort_flag);
                        if (!ok) break;
                        tc_fence_after_sync();
                    }
                    issue_dq();
                    mma_commit(&bars[Cfg::kDqFull]);
                    if (more && kDqAliasesT2) {
                        // the tile sits in T2's columns: dP^T(it+1) may only follow its read-out
                        ok = mbar_wait(&bars[Cfg::kDqRead], (uint32_t)it & 1u, abort_flag);
                        if (!ok) break;
                        tc_fence_after_sync();
                    }
                }
                if (KS && more) {
                    ok = mbar_wait(&bars[kWReady + nws], nwph & 1u, abort_flag);
                    if (!ok) break;
                    tc_fence_after_sync();
                    issue_t(tT2, sY_u, nxt_w, idesc_t2);
                    mma_commit(&bars[Cfg::kT2Full]);
                }
                us = nus; uph = nuph; ws = nws; wph = nwph;
            }
            if (ok) mma_commit(&bars[Cfg::kAccDone]);
        }
        __syncwarp();
      } else if (STREAM_CONV) {
        // ---------------------------------------------------------------- warps 18-19: streamed tiles -> fp16
        // the producer's walk; a tile is touched between its arrival (U_full / W_full) and its first
        // reader (the MMAs wait for U_conv / W_conv).  dO tiles are normalised on the way.
        const int ct = (warp - kTmaWarp - 1) * 32 + lane;
        int us = 0, ws = 0;
        uint32_t uph = 0, wph = 0;
        for (int it = 0; it < n_iter; ++it) {
            bool ok = mbar_wait(&bars[Cfg::kUFull + us], uph & 1u, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            convert_tile_bf16_to_f16<false>(sU + us * TILE, TILE, ct, 64, 1.f);
            fence_proxy_async_smem();
            mbar_arrive_warp(&bars[Cfg::kUConv + us]);
            if (KS) {
                ok = mbar_wait(&bars[Cfg::kWFull + ws], wph & 1u, abort_flag);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                convert_tile_bf16_to_f16<true>(sW + ws * TILE, TILE, ct, 64, sc.do_mul);
                fence_proxy_async_smem();
                mbar_arrive_warp(&bars[Cfg::kWConv + ws]);
            }
            if (++us == UST) { us = 0; ++uph; }
            if (++ws == WST) { ws = 0; ++wph; }
        }
      }
    } else {
        // ---------------------------------------------------------------- P / dS and epilogue
        if constexpr (kMoveRegs) asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsElementwiseMoved));
        constexpr int NLD = CPT / 32;                          // 32-column TMEM loads per thread and phase
        const int wg = warp >> 2;                              // which CPT-column slice
        const int r = (warp & 3) * 32 + lane;                  // TMEM lane = row of T1/T2
        const int cb = wg * CPT;
        const int tid = wg * 128 + r;                          // 0 .. 128*NWG-1
        const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
        const int row_g = tile * kTile + r;                    // MODE 0: key index; MODE 1: query index
        constexpr bool drop = DROP != 0;
        float my_nlse2 = 0.f, my_ndelta = 0.f;      // -lse*log2(e) and -delta of my query row (MODE 1)
        if (MODE == 1) {
            const int64_t off = ((int64_t)b * a.H + head_x) * a.nq_pad + row_g;
            my_nlse2 = a.lse2[off];
            my_ndelta = a.delta[off];
            if (ROWFORM) {
                // the vectors are staged for the key-stationary kernels: take the row exponent out again
                const int e_i = (int)a.erow[off];
                my_nlse2 -= (float)e_i;            // -inf in the padding stays -inf
                my_ndelta *= pow2i(e_i);
            }
        }
        // dS' = P' o (dP * tt_mul o Z + (-delta) * nd_mul): see "number formats" above
        const uint64_t ttm2 = f2_pack(sc.tt_mul, sc.tt_mul), ndm2 = f2_pack(sc.nd_mul, sc.nd_mul);
        const float zk = a.inv_keep * sc.tt_mul;
        const uint64_t ladd2 = f2_pack(sc.l_add, sc.l_add);
        my_ndelta *= sc.nd_mul;
        bool ok = true;
        if (XY_CONV && n_iter > 0) {
            // the stationary tiles, once per CTA: K_j and V_j, or Q_i (dO_i is only ever multiplied
            // with the bf16 V_j tiles and stays as it is)
            ok = mbar_wait(&bars[Cfg::kXYFull], 0u, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (ok) {
                convert_tile_bf16_to_f16<false>(sX, (KS ? 2 : 1) * TILE, tid, 128 * NWG, 1.f);   // Y follows X
                fence_proxy_async_smem();
                mbar_arrive_warp(&bars[Cfg::kXYConv]);
                if (K_COPY && tid == 0 && mbar_wait(&bars[Cfg::kXYConv], 0u, abort_flag)) {
                    // the fp16 K tile is what the dQ kernel streams: keep a copy (rows beyond Nk are clipped)
#pragma unroll
                    for (int bx = 0; bx < Cfg::kNBox; ++bx)
                        tma_store_4d(&map_aux, sX + bx * kBoxBytes, bx * 64, head_x, tile * kTile, b);
                    tma_store_commit();       // read out before the kernel ends: the epilogue waits for all groups
                }
            }
        }

        // fused kernel: add the dQ tile of step `jt` (queries on the TMEM lanes, my D / NWG columns)
        // to the fp32 sums in global memory; the order of additions across CTAs is not fixed
        auto drain_dq = [&](int jt, int q_tile, int head_q) -> bool {
            constexpr int DQC = D / NWG;
            bool good = mbar_wait(&bars[Cfg::kDqFull], (uint32_t)jt & 1u, abort_flag);
            good = __all_sync(0xffffffffu, good);
            if (!good) return false;
            tc_fence_after_sync();
            uint32_t acc[DQC];
            if constexpr (DQC == 32) tmem_ld_32x32(tDq + lane_off + (uint32_t)(wg * DQC), acc);
            else                     tmem_ld_32x16(tDq + lane_off + (uint32_t)(wg * DQC), acc);
            tmem_wait_ld();
            tc_fence_before_sync();
            mbar_arrive_warp(&bars[Cfg::kDqRead]);
            float* dst = a.dq_acc + (((int64_t)b * a.H + head_q) * (a.nq_pad / kTile) + q_tile) * (int64_t)(kTile * D) +
                         ((int64_t)(wg * (DQC / 4)) * kTile + r) * 4;
#pragma unroll
            for (int v = 0; v < DQC / 4; ++v)
                red_add_v4_f32(dst + (int64_t)v * kTile * 4, __uint_as_float(acc[4 * v]), __uint_as_float(acc[4 * v + 1]),
                               __uint_as_float(acc[4 * v + 2]), __uint_as_float(acc[4 * v + 3]));
            return true;
        };

        int qi = 0, hg = 0;                 // step within the query head, query heads done (key-stationary)
        int prev_tile = 0, prev_head = 0;   // query tile and head of the previous step
        for (int it = 0; it < n_iter; ++it) {
            const int strm_tile = (KS) ? q_tile_of(qi) : it;     // query tile (0) / key tile (1)
            const int col_g0 = strm_tile * kTile + cb;                          // global index of my first column
            const int head_q = (KS) ? head_x * group + hg : head_x;
            const uint32_t bh = dropout_column(a.rng, b, head_q);
            // key-stationary: -lse*log2(e) and -delta of this step's 128 queries (slot it & 1)
            const float* lse_s = sVec + (it & 1) * 256;
            const float* del_s = lse_s + 128;

            // ---- dropout keep bits of my CPT columns (bit c of kb[c / 32])
            uint32_t kb[2] = {0xFFFFFFFFu, 0xFFFFFFFFu};
            if (drop) {
                kb[0] = 0u; kb[1] = 0u;
                if constexpr (DROP == 2) {
                    static_assert(CPT % 32 == 0, "a thread's columns are whole words of the bit buffer");
                    if (MODE == 1) {
                        // my query row's bits for this key tile: the words of my CPT columns
                        const uint32_t* w = reinterpret_cast<const uint32_t*>(
                            a.bits_q + ((int64_t)(b * a.H + head_q) * (a.nk_pad / kTile) + strm_tile) * a.nq_pad + row_g);
#pragma unroll
                        for (int g = 0; g < CPT / 32; ++g) kb[g] = w[cb / 32 + g];
                    } else if (FUSED) {
                        // my key row's bits for this query tile, 32 queries a word
                        const uint32_t* w = a.bits_k + (((int64_t)(b * a.H + head_q) * (a.nq_pad / kTile) + strm_tile) * 4 +
                                                        cb / 32) * (int64_t)a.nk_pad + row_g;
#pragma unroll
                        for (int g = 0; g < CPT / 32; ++g) kb[g] = w[(int64_t)g * a.nk_pad];
                    }
                } else if (MODE == 1) {
#pragma unroll
                    for (int g = 0; g < CPT / 16; ++g) {
                        const uint32_t w = dropout_keep_bits(a.key, bh, (uint32_t)row_g, (uint32_t)((col_g0 >> 4) + g),
                                                             a.drop_thr);
                        kb[g >> 1] |= w << (16 * (g & 1));
                    }
                } else {
                    // keys are rows here: build the tile's masks cooperatively, query-major, then read
                    // one bit per (query column, my key row)
                    constexpr int PER = 8 / NWG;               // 16-key blocks each thread generates
                    uint16_t* mbuf = sMask + (it & 1) * (128 * 8);
                    const int ql = tid & 127, jb0 = (tid >> 7) * PER;
#pragma unroll
                    for (int g = 0; g < PER; ++g)
                        mbuf[ql * 8 + jb0 + g] = (uint16_t)dropout_keep_bits(
                            a.key, bh, (uint32_t)(strm_tile * kTile + ql), (uint32_t)(tile * 8 + jb0 + g), a.drop_thr);
                    mbar_arrive_warp(&bars[Cfg::kMask]);
                    ok = mbar_wait(&bars[Cfg::kMask], (uint32_t)it & 1u, abort_flag);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    if (FUSED) {      // (the fragment-layout phases read their keep bits from mbuf themselves)
                        const int jw = r >> 4, jbit = r & 15;
#pragma unroll
                        for (int c = 0; c < CPT; ++c)
                            kb[c >> 5] |= (((uint32_t)mbuf[(cb + c) * 8 + jw] >> jbit) & 1u) << (c & 31);
                    }
                }
            }

            if constexpr (MODE == 0) {
            // ---- dK/dV kernel, fragment layout: a thread holds 4 rows x 8 columns of its warp's
            // 32 x 32 block (rows lane/4 + {0, 8, 16, 24}, columns 8j + 2(lane%4) + {0, 1}, j = 0..3) instead
            // of 1 row x 32 columns, so it needs the -lse / -delta values of 8 query columns, four 8-byte
            // loads that one wavefront serves, instead of 32 values through eight broadcast 16-byte loads.
            const int lq = lane & 3, lr = lane >> 2;
            const int rbase = (warp & 3) * 32 + lr;                 // my first row inside the tile
            // DROP = 2: one word of keep bits per key row of mine, asked for before the wait for S^T
            uint32_t kwr[2][2] = {{0u, 0u}, {0u, 0u}};
            if constexpr (DROP == 2) {
                const uint32_t* w = a.bits_k + (((int64_t)(b * a.H + head_q) * (a.nq_pad / kTile) + strm_tile) * 4 +
                                                cb / 32) * (int64_t)a.nk_pad + tile * kTile + rbase;
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                    for (int k = 0; k < 2; ++k) kwr[h][k] = w[16 * h + 8 * k];
            }
            ok = mbar_wait(&bars[Cfg::kT1Full], (uint32_t)it & 1u, abort_flag);
            if (ok) ok = mbar_wait(&bars[Cfg::kVFull + (it & 1)], (uint32_t)(it >> 1) & 1u, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after_sync();
            const uint32_t t_lo = lane_off + cb, t_hi = lane_off + (16u << 16) + cb;
            // element (h, j, k, e): row rbase + 16h + 8k, column 8j + 2lq + e, register [h][4j + 2k + e]
            uint32_t pf[2][16];
            tmem_ld_16x256b_x4(tT1 + t_lo, pf[0]);
            tmem_ld_16x256b_x4(tT1 + t_hi, pf[1]);
            tmem_wait_ld();
            uint32_t kbits = 0xFFFFFFFFu;                           // keep bit of element (h, j, k, e): bit 16h + 4j + 2k + e
            if constexpr (DROP == 2) {
                // shifted so that bit 8j + e is my column 8j + 2lq + e
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                    for (int k = 0; k < 2; ++k) kwr[h][k] >>= ((cb & 31) + 2 * lq);
            } else if (drop) {
                const uint16_t* mbuf = sMask + (it & 1) * (128 * 8);
                kbits = 0u;
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                    for (int j = 0; j < 4; ++j)
#pragma unroll
                        for (int k = 0; k < 2; ++k)
#pragma unroll
                            for (int e = 0; e < 2; ++e) {
                                const int row = rbase + 16 * h + 8 * k, col = cb + 8 * j + 2 * lq + e;
                                kbits |= (((uint32_t)mbuf[col * 8 + (row >> 4)] >> (row & 15)) & 1u) << (16 * h + 4 * j + 2 * k + e);
                            }
            }
            const uint64_t sc2 = f2_pack(a.scale_log2, a.scale_log2);
            // key row > query column + shift is hidden: only tiles the mask's edge crosses need the test
            const bool diag = a.causal && strm_tile * kTile + a.shift < tile * kTile + kTile - 1;
            const bool tail = tile * kTile + kTile > nk;            // the tile holds padding keys
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
                uint32_t pk[2][4];                                  // [h][2j' + k], j' = j - 2hf
#pragma unroll
                for (int jj = 0; jj < 2; ++jj) {
                    const int j = 2 * hf + jj;
                    if (!drop && hf == 1 && jj == 0) {
                        // hand the first half over before the second is computed, so that its MMAs are done
                        // when the second half arrives (dK/dV 0.971 -> 0.933 ms at B4 N4096 H32 D128: the chain
                        // MMA -> threads -> MMA feels every cycle).  With dropout the threads are the slower
                        // side and the wait for the stores just issued costs more than it gains (1.24 against
                        // 1.22 ms at B32 N2048 H16 D64): there the hand-off stays behind the second half's math.
                        tmem_wait_st();
                        tc_fence_before_sync();
                        mbar_arrive_warp(&bars[Cfg::kPHalf]);
                    }
                    uint64_t L = *reinterpret_cast<const uint64_t*>(lse_s + cb + 8 * j + 2 * lq);
                    if (ROWFORM) L = f2_add(L, ladd2);
#pragma unroll
                    for (int h = 0; h < 2; ++h)
#pragma unroll
                        for (int k = 0; k < 2; ++k) {
                            const int i0 = 4 * j + 2 * k;
                            float x0, x1;
                            f2_unpack(f2_fma(f2_pack(__uint_as_float(pf[h][i0]), __uint_as_float(pf[h][i0 + 1])), sc2, L), x0, x1);
                            pf[h][i0] = __float_as_uint(ex2(x0));
                            pf[h][i0 + 1] = __float_as_uint(ex2(x1));
                        }
                }
                if (diag || tail) {
                    // one branch for the whole half: the diagonal tile and a tile with padding keys are rare
#pragma unroll
                    for (int jj = 0; jj < 2; ++jj)
#pragma unroll
                        for (int h = 0; h < 2; ++h)
#pragma unroll
                            for (int k = 0; k < 2; ++k) {
                                const int j = 2 * hf + jj, i0 = 4 * j + 2 * k;
                                const int row_k = tile * kTile + rbase + 16 * h + 8 * k;
                                const int col = col_g0 + 8 * j + 2 * lq;
                                // query columns below `lim` do not see this key row: all of them for a
                                // padding key, those with column + shift < row under the mask's edge
                                const int lim = (tail && row_k >= nk) ? 0x7fffffff : (diag ? row_k - a.shift : -0x7fffffff);
                                if (col < lim) pf[h][i0] = 0u;
                                if (col + 1 < lim) pf[h][i0 + 1] = 0u;
                            }
                }
#pragma unroll
                for (int jj = 0; jj < 2; ++jj)
#pragma unroll
                    for (int h = 0; h < 2; ++h)
#pragma unroll
                        for (int k = 0; k < 2; ++k) {
                            const int i0 = 4 * (2 * hf + jj) + 2 * k;
                            float z0 = __uint_as_float(pf[h][i0]), z1 = __uint_as_float(pf[h][i0 + 1]);
                            if (drop) {
                                const uint32_t kw = DROP == 2 ? kwr[h][k] >> (8 * (i0 >> 2)) : kbits >> (16 * h + i0);
                                if (!(kw & 1u)) z0 = 0.f;
                                if (!(kw & 2u)) z1 = 0.f;
                            }
                            pk[h][2 * jj + k] = pack2<false>(z0, z1);
                        }
                if (drop && hf == 1) {
                    tmem_wait_st();
                    tc_fence_before_sync();
                    mbar_arrive_warp(&bars[Cfg::kPHalf]);
                }
                tmem_st_16x128b_x2(tT1 + t_lo + hf * 8, pk[0]);
                tmem_st_16x128b_x2(tT1 + t_hi + hf * 8, pk[1]);
            }
            tmem_wait_st();
            tc_fence_before_sync();
            mbar_arrive_warp(&bars[Cfg::kPReady]);

            ok = mbar_wait(&bars[Cfg::kT2Full], (uint32_t)it & 1u, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after_sync();
            {
                uint32_t df[2][16];
                tmem_ld_16x256b_x4(tT2 + t_lo, df[0]);
                tmem_ld_16x256b_x4(tT2 + t_hi, df[1]);
                tmem_wait_ld();
#pragma unroll
                for (int hf = 0; hf < 2; ++hf) {
                    uint32_t pk[2][4];
#pragma unroll
                    for (int jj = 0; jj < 2; ++jj) {
                        const int j = 2 * hf + jj;
                        if (!drop && hf == 1 && jj == 0) {
                            tmem_wait_st();                        // the first half, as for P above
                            tc_fence_before_sync();
                            mbar_arrive_warp(&bars[Cfg::kDsHalf]);
                        }
                        const uint64_t nd = f2_mul(*reinterpret_cast<const uint64_t*>(del_s + cb + 8 * j + 2 * lq), ndm2);
#pragma unroll
                        for (int h = 0; h < 2; ++h)
#pragma unroll
                            for (int k = 0; k < 2; ++k) {
                                const int i0 = 4 * j + 2 * k;
                                const uint64_t dp = f2_pack(__uint_as_float(df[h][i0]), __uint_as_float(df[h][i0 + 1]));
                                uint64_t tt;
                                if (drop) {
                                    const uint32_t kw = DROP == 2 ? kwr[h][k] >> (8 * j) : kbits >> (16 * h + i0);
                                    tt = f2_fma(dp, f2_pack((kw & 1u) ? zk : 0.f, (kw & 2u) ? zk : 0.f), nd);
                                } else {
                                    tt = f2_fma(dp, ttm2, nd);
                                }
                                float d0, d1;
                                f2_unpack(f2_mul(f2_pack(__uint_as_float(pf[h][i0]), __uint_as_float(pf[h][i0 + 1])), tt), d0, d1);
                                pk[h][2 * jj + k] = pack2<false>(d0, d1);
                            }
                    }
                    if (drop && hf == 1) {
                        tmem_wait_st();
                        tc_fence_before_sync();
                        mbar_arrive_warp(&bars[Cfg::kDsHalf]);
                    }
                    tmem_st_16x128b_x2(tT2 + t_lo + hf * 8, pk[0]);
                    tmem_st_16x128b_x2(tT2 + t_hi + hf * 8, pk[1]);
                }
                tmem_wait_st();
            }
            tc_fence_before_sync();
            mbar_arrive_warp(&bars[Cfg::kDsReady]);
            } else {
            // ---- one row and 32 columns per thread: the query-stationary kernel (lse and delta are
            // per-thread scalars there), and the one-kernel backward, whose dS^T tile for the dQ MMA is
            // written with 16-byte stores from this layout (with the fragment layout above it measured
            // 5-10 % slower)
            // ---- phase A: P from T1
            ok = mbar_wait(&bars[Cfg::kT1Full], (uint32_t)it & 1u, abort_flag);
            if (KS && ok) ok = mbar_wait(&bars[Cfg::kVFull + (it & 1)], (uint32_t)(it >> 1) & 1u, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after_sync();
            uint32_t pr[NLD][32];      // P of my columns (fp32 bits), kept for phase B
#define PF(c) __uint_as_float(pr[(c) >> 5][(c) & 31])
#define PSET(c, x) pr[(c) >> 5][(c) & 31] = __float_as_uint(x)
#pragma unroll
            for (int q = 0; q < NLD; ++q) tmem_ld_32x32(tT1 + lane_off + cb + q * 32, pr[q]);
            tmem_wait_ld();
            if (!KS) {
                // query-stationary: P stays in registers, so S's columns are free for S(it+1) from here on
                tc_fence_before_sync();
                mbar_arrive_warp(&bars[Cfg::kPReady]);
            }
            const uint64_t sc2 = f2_pack(a.scale_log2, a.scale_log2);
            if (KS) {
                // P = 2^(S*c - lse): the staged vector holds -lse*log2(e), two columns per 64-bit word.
                // Two halves of CPT / 2 columns: the first is packed, stored to TMEM and handed to the
                // MMA warp (dV can start on it) while the second is computed.
                static_assert(CPT == 32, "the half hand-off is written for 32 columns per thread");
                const ulonglong2* l2 = reinterpret_cast<const ulonglong2*>(lse_s + cb);
                const bool diag = a.causal && strm_tile * kTile + a.shift < tile * kTile + kTile - 1;
#pragma unroll
                for (int hf = 0; hf < 2; ++hf) {
                    if (hf == 1) {
                        // hand the first half over before the second is computed: its MMAs are then done
                        // when the second half arrives (the chain MMA -> threads -> MMA feels every cycle)
                        tmem_wait_st();
                        tc_fence_before_sync();
                        mbar_arrive_warp(&bars[Cfg::kPHalf]);
                    }
#pragma unroll
                    for (int c4 = hf * (CPT / 8); c4 < (hf + 1) * (CPT / 8); ++c4) {
                        ulonglong2 L = l2[c4];
                        if (ROWFORM) { L.x = f2_add(L.x, ladd2); L.y = f2_add(L.y, ladd2); }
                        float x0, x1, x2, x3;
                        f2_unpack(f2_fma(f2_pack(PF(c4 * 4 + 0), PF(c4 * 4 + 1)), sc2, L.x), x0, x1);
                        f2_unpack(f2_fma(f2_pack(PF(c4 * 4 + 2), PF(c4 * 4 + 3)), sc2, L.y), x2, x3);
                        PSET(c4 * 4 + 0, ex2(x0));
                        PSET(c4 * 4 + 1, ex2(x1));
                        PSET(c4 * 4 + 2, ex2(x2));
                        PSET(c4 * 4 + 3, ex2(x3));
                    }
                    if (diag) {
                        const int hidden = row_g - col_g0 - a.shift;   // my first `hidden` columns: query + shift < key
#pragma unroll
                        for (int c = hf * (CPT / 2); c < (hf + 1) * (CPT / 2); ++c)
                            if (c < hidden) PSET(c, 0.f);
                    }
                    if (row_g >= nk) {                    // a padding key inside a live tile (or beyond Nk)
#pragma unroll
                        for (int c = hf * (CPT / 2); c < (hf + 1) * (CPT / 2); ++c) PSET(c, 0.f);
                    }
                    uint32_t pk[CPT / 4];
#pragma unroll
                    for (int e = 0; e < CPT / 4; ++e) {
                        const int c = hf * (CPT / 2) + 2 * e;
                        float x0 = PF(c), x1 = PF(c + 1);
                        if (drop) {
                            if (!((kb[c >> 5] >> (c & 31)) & 1u)) x0 = 0.f;
                            if (!((kb[(c + 1) >> 5] >> ((c + 1) & 31)) & 1u)) x1 = 0.f;
                        }
                        pk[e] = pack2<false>(x0, x1);
                    }
                    tmem_st_32x8(tT1 + lane_off + cb + hf * (CPT / 4), pk);
                }
                tmem_wait_st();
            } else {
                const uint64_t neg2 = f2_pack(my_nlse2, my_nlse2);
#pragma unroll
                for (int c = 0; c < CPT; c += 2) {
                    float x0, x1;
                    f2_unpack(f2_fma(f2_pack(PF(c), PF(c + 1)), sc2, neg2), x0, x1);
                    // a quarter of the exponentials as a polynomial on the FMA pipes (this kernel keeps the
                    // special-function unit busiest; measured 0.7 % over the backward, half: 0.2 %)
                    if (((c >> 1) & 3) == 0) {
                        float p0, p1;
                        ex2_poly2(x0, x1, p0, p1);
                        PSET(c, p0);
                        PSET(c + 1, p1);
                    } else {
                        PSET(c, ex2(x0));
                        PSET(c + 1, ex2(x1));
                    }
                }
                const bool diag = a.causal && strm_tile * kTile + kTile - 1 > tile * kTile + a.shift;
                if (diag || strm_tile * kTile + kTile > nk) {
                    // my row sees my first `seen` columns: keys below the count, at most row + shift
                    int seen = nk - col_g0;
                    if (diag && row_g + a.shift + 1 - col_g0 < seen) seen = row_g + a.shift + 1 - col_g0;
#pragma unroll
                    for (int c = 0; c < CPT; ++c)
                        if (c >= seen) PSET(c, 0.f);
                }
            }
            if (KS) {
                tc_fence_before_sync();
                mbar_arrive_warp(&bars[Cfg::kPReady]);
            }

            if (FUSED && it > 0) {
                // dQ of the previous step: its MMAs ran while phase A above did
                ok = drain_dq(it - 1, prev_tile, prev_head);
                if (!ok) break;
            }

            // ---- phase B: dS from T2
            // query-stationary: dP / dS alternate between two buffers, each with its own barriers
            const bool odd_buf = !KS && (it & 1);
            const uint32_t tD = odd_buf ? tAcc2 : tT2;
            const int b_half = odd_buf ? Cfg::kPHalf : Cfg::kDsHalf, b_ready = odd_buf ? Cfg::kDqRead : Cfg::kDsReady;
            ok = KS ? mbar_wait(&bars[Cfg::kT2Full], (uint32_t)it & 1u, abort_flag)
                    : mbar_wait(&bars[odd_buf ? Cfg::kT1Full + 1 : Cfg::kT2Full], (uint32_t)(it >> 1) & 1u, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after_sync();
            {
                uint32_t dr[NLD][32];
#pragma unroll
                for (int q = 0; q < NLD; ++q) tmem_ld_32x32(tD + lane_off + cb + q * 32, dr[q]);
                tmem_wait_ld();
                // dS = P o (dP o Z - delta); the staged vector holds -delta.  Two halves, as in phase A:
                // the first is stored and handed over while the second is computed.
                const ulonglong2* d2 = reinterpret_cast<const ulonglong2*>(del_s + cb);
                const uint64_t my_nd2 = f2_pack(my_ndelta, my_ndelta);
#pragma unroll
                for (int hf = 0; hf < 2; ++hf) {
                    uint32_t pk[CPT / 4];
                    if (hf == 1) {
                        tmem_wait_st();                            // the first half, stored just now
                        tc_fence_before_sync();
                        mbar_arrive_warp(&bars[b_half]);
                    }
#pragma unroll
                    for (int c4 = hf * (CPT / 8); c4 < (hf + 1) * (CPT / 8); ++c4) {
                        ulonglong2 nd;
                        if (KS) { nd = d2[c4]; nd.x = f2_mul(nd.x, ndm2); nd.y = f2_mul(nd.y, ndm2); }
                        else { nd.x = my_nd2; nd.y = my_nd2; }
                        const int c = c4 * 4;
                        uint64_t dpa = f2_pack(__uint_as_float(dr[c >> 5][c & 31]), __uint_as_float(dr[c >> 5][(c + 1) & 31]));
                        uint64_t dpb = f2_pack(__uint_as_float(dr[c >> 5][(c + 2) & 31]), __uint_as_float(dr[c >> 5][(c + 3) & 31]));
                        uint64_t ta, tb;
                        if (drop) {
                            // dropped entries: dS = P o (-delta), selected after the FMA
                            const uint32_t kw = kb[c >> 5] >> (c & 31);
                            const uint64_t zk2 = f2_pack(zk, zk);
                            float t0, t1, t2, t3, n0, n1, n2, n3;
                            f2_unpack(f2_fma(dpa, zk2, nd.x), t0, t1);
                            f2_unpack(f2_fma(dpb, zk2, nd.y), t2, t3);
                            f2_unpack(nd.x, n0, n1);
                            f2_unpack(nd.y, n2, n3);
                            ta = f2_pack((kw & 1u) ? t0 : n0, (kw & 2u) ? t1 : n1);
                            tb = f2_pack((kw & 4u) ? t2 : n2, (kw & 8u) ? t3 : n3);
                        } else {
                            ta = f2_fma(dpa, ttm2, nd.x);
                            tb = f2_fma(dpb, ttm2, nd.y);
                        }
                        float d0, d1, d2v, d3;
                        f2_unpack(f2_mul(f2_pack(PF(c), PF(c + 1)), ta), d0, d1);
                        f2_unpack(f2_mul(f2_pack(PF(c + 2), PF(c + 3)), tb), d2v, d3);
                        pk[(c4 - hf * (CPT / 8)) * 2 + 0] = pack2<false>(d0, d1);
                        pk[(c4 - hf * (CPT / 8)) * 2 + 1] = pack2<false>(d2v, d3);
                    }
                    tmem_st_32x8(tD + lane_off + cb + hf * (CPT / 4), pk);
                    if (FUSED) {
                        // the same dS^T values as a shared-memory tile [key row][query], 64-query boxes with
                        // the 128-byte swizzle: the A operand (MN-major) of the dQ MMA.  The previous
                        // step's dQ MMA has finished reading it: its completion was awaited in drain_dq.
#pragma unroll
                        for (int v = 0; v < CPT / 16; ++v) {
                            const int q0 = cb + hf * (CPT / 2) + v * 8;                 // first of 8 queries
                            uint8_t* dst = sDs + (q0 >> 6) * kBoxBytes + r * 128 + ((((q0 & 63) >> 3) ^ (r & 7)) << 4);
                            *reinterpret_cast<uint4*>(dst) = make_uint4(pk[4 * v], pk[4 * v + 1], pk[4 * v + 2], pk[4 * v + 3]);
                        }
                    }
                }
                if (FUSED) fence_proxy_async_smem();
                tmem_wait_st();
            }
#undef PF
#undef PSET
            tc_fence_before_sync();
            mbar_arrive_warp(&bars[b_ready]);
            }
            if (KS) mbar_arrive_warp(&bars[Cfg::kVEmpty + (it & 1)]);      // this step's lse / delta rows are read
            prev_tile = strm_tile; prev_head = head_q;
            if (++qi == n_per_head) { qi = 0; ++hg; }
        }

        if (FUSED && n_iter > 0 && ok) ok = drain_dq(n_iter - 1, prev_tile, prev_head);

        // ---- epilogue: accumulators -> 16-bit -> swizzled staging -> TMA store
        if (n_iter > 0 && ok) ok = mbar_wait(&bars[Cfg::kAccDone], 0u, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (ok) {
            tc_fence_after_sync();
            constexpr int kCols = D / NWG;                     // my share of the D accumulator columns: 16..64
            constexpr int kOuts = (KS) ? 2 : 1;
#pragma unroll
            for (int o = 0; o < kOuts; ++o) {
                const uint32_t tacc = (o == 0 ? tAcc1 : tAcc2) + lane_off + (uint32_t)(wg * kCols);
                const float mul = (o == 0) ? sc.acc1_mul : sc.acc2_mul;
                uint8_t* stage = sU + o * TILE;                // the U ring is idle once all MMAs completed
#pragma unroll
                for (int c0 = 0; c0 < kCols; c0 += 32) {
                    constexpr int kN = kCols < 32 ? kCols : 32;
                    uint32_t acc[kN];
                    if (n_iter > 0) {
                        if constexpr (kN == 32) tmem_ld_32x32(tacc + c0, acc);
                        else                    tmem_ld_32x16(tacc + c0, acc);
                        tmem_wait_ld();
                    } else {
#pragma unroll
                        for (int c = 0; c < kN; ++c) acc[c] = 0u;    // no query sees this key tile
                    }
#pragma unroll
                    for (int g = 0; g < kN / 8; ++g) {
                        uint4 v4;
                        v4.x = pack2<BF16>(__uint_as_float(acc[g * 8 + 0]) * mul, __uint_as_float(acc[g * 8 + 1]) * mul);
                        v4.y = pack2<BF16>(__uint_as_float(acc[g * 8 + 2]) * mul, __uint_as_float(acc[g * 8 + 3]) * mul);
                        v4.z = pack2<BF16>(__uint_as_float(acc[g * 8 + 4]) * mul, __uint_as_float(acc[g * 8 + 5]) * mul);
                        v4.w = pack2<BF16>(__uint_as_float(acc[g * 8 + 6]) * mul, __uint_as_float(acc[g * 8 + 7]) * mul);
                        const int col = wg * kCols + c0 + g * 8;
                        const int chunk = (col & 63) >> 3;
                        uint8_t* dst = stage + (col >> 6) * kBoxBytes + r * 128 + ((chunk ^ (r & 7)) << 4);
                        *reinterpret_cast<uint4*>(dst) = v4;
                    }
                }
            }
            fence_proxy_async_smem();
            mbar_arrive_warp(&bars[Cfg::kEpi]);
            if (tid == 0 && mbar_wait(&bars[Cfg::kEpi], 0u, abort_flag)) {
#pragma unroll
                for (int bx = 0; bx < Cfg::kNBox; ++bx) {
                    tma_store_4d(&map_out1, sU + bx * kBoxBytes, bx * 64, head_x, tile * kTile, b);
                    if (KS)
                        tma_store_4d(&map_out2, sU + TILE + bx * kBoxBytes, bx * 64, head_x, tile * kTile, b);
                }
                tma_store_commit();
                tma_store_wait_read<0>();   // the staging tile has been read; the writes complete on their own
            }
        }
    }

    if (K_COPY && threadIdx.x == 0) tma_store_wait_read<0>();   // the K copy's source tile (also when unwinding)
    tc_fence_before_sync();
    __syncthreads();
    if (warp == kMmaWarp) tmem_dealloc(tmem, 512);
    if (threadIdx.x == 0 && *abort_flag) report_status(a.status, 2 + MODE);
    // the end of this grid must still mean the end of the dK/dV grid before it in the stream
    if (MODE == 1) grid_dependency_wait();
}

// Largest magnitude among the eight 16-bit values of a 16-byte piece, folded into a running maximum
// of magnitude bit patterns (two per word; for fp16 and bf16 alike a larger magnitude is a larger
// unsigned pattern).
__device__ __forceinline__ uint32_t absmax16_acc(uint32_t m, const uint4& v) {
    asm("max.u16x2 %0, %0, %1;" : "+r"(m) : "r"(v.x & 0x7FFF7FFFu));
    asm("max.u16x2 %0, %0, %1;" : "+r"(m) : "r"(v.y & 0x7FFF7FFFu));
    asm("max.u16x2 %0, %0, %1;" : "+r"(m) : "r"(v.z & 0x7FFF7FFFu));
    asm("max.u16x2 %0, %0, %1;" : "+r"(m) : "r"(v.w & 0x7FFF7FFFu));
    return m;
}
// Block-wide maximum of those patterns, as a float, folded into *slot (an fp32 bit pattern; for
// non-negative floats the unsigned order is the numeric order, so atomicMax on the bits is exact).
template <typename T>
__device__ __forceinline__ void absmax16_commit(uint32_t m, float* slot, uint32_t* red) {
    m = max(m & 0xFFFFu, m >> 16);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, off));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < (int)(blockDim.x >> 5); ++w) m = max(m, red[w]);
        const unsigned short bits = (unsigned short)m;
        const float f = to_f32<T>(*reinterpret_cast<const T*>(&bits));
        atomicMax(reinterpret_cast<uint32_t*>(slot), __float_as_uint(f));
    }
}

// Preprocess launch.  Blocks [0, n_row_blocks): negated delta and the shifted, negated, scaled lse (the
// main kernels add them), and max |dO| of the block's column.  D / 8 lanes share one (b, h, padded query
// row), 16 bytes of O and dO each, so a warp covers 256 / D rows; a block's rows lie in one (b, h).
// Blocks beyond: max |V| over a slab of one (b, K/V head) column's visible keys.
// ranges[(b * Hkv + hk) * 2 + {0, 1}] = max |dO| over the K/V head's query heads, max |V|; zeroed before.
// COPIES (bf16): also the fp16 copies the main kernels stream, dense (B, Nq, H, D): Q as it is, dO row
// by row normalised to max < 2^15 by 2^-e_i, with e_i kept in `erow` and folded into the two vectors
// (lse' = kPShift - lse*log2(e) + e_i, -delta * 2^-e_i: the "row form" of make_scales).
struct PreprocessCopies {
    const void* o_lo; int64_t l_sb, l_sn, l_sh;     // optional residual of O (any dtype)
    const void* q; int64_t q_sb, q_sn, q_sh;
    uint16_t* q16; uint16_t* do16; float* erow;
};
template <typename T, int D, bool COPIES>
__global__ void __launch_bounds__(256)
bwd_preprocess_kernel(const T* __restrict__ o, const T* __restrict__ d_o, const float* __restrict__ lse,
                      float* __restrict__ lse2, float* __restrict__ delta, float* __restrict__ ranges,
                      int B, int Nq, int H, int Hkv, int nq_pad,
                      int64_t o_sb, int64_t o_sn, int64_t o_sh, int64_t g_sb, int64_t g_sn, int64_t g_sh,
                      const T* __restrict__ v, int64_t v_sb, int64_t v_sn, int64_t v_sh, int Nk,
                      const int32_t* __restrict__ kv_len, int n_row_blocks, int v_slabs, const PreprocessCopies cp) {
    constexpr int LPR = D / 8;                 // lanes per row
    constexpr int RPW = 32 / LPR;              // rows per warp
    constexpr int kVRows = 256;                // keys per slab of the V scan
    __shared__ uint32_t red[8];
    const int lane = threadIdx.x & 31, sub = lane % LPR;
    if ((int)blockIdx.x >= n_row_blocks) {
        const int vb = (int)blockIdx.x - n_row_blocks;
        const int slab = vb % v_slabs, col = vb / v_slabs;          // col = b * Hkv + hk
        const int hk = col % Hkv, b = col / Hkv;
        const int nk = kv_len_of(kv_len, b, Nk);
        uint32_t m = 0u;
        const int j_end = min(nk, (slab + 1) * kVRows);
        for (int j = slab * kVRows + (int)(threadIdx.x / LPR); j < j_end; j += 256 / LPR)
            m = absmax16_acc(m, *reinterpret_cast<const uint4*>(v + b * v_sb + (int64_t)j * v_sn + hk * v_sh + sub * 8));
        absmax16_commit<T>(m, ranges + 2 * (int64_t)col + 1, red);
        return;
    }
    // a block takes one 128-row tile of one (b, h): kPasses passes of 256 / LPR rows, a pass's loads
    // issued together; one reduction of max |dO| per block
    constexpr int kRowsPerPass = 8 * RPW;
    constexpr int kPasses = 128 / kRowsPerPass;
    const int tiles_per_col = nq_pad / 128;
    const int64_t bh = (int64_t)blockIdx.x / tiles_per_col;
    const int i0 = ((int)blockIdx.x - (int)(bh * tiles_per_col)) * 128 + (int)(threadIdx.x >> 5) * RPW + lane / LPR;
    const int h = (int)(bh % H), b = (int)(bh / H);
    const T* op = o + b * o_sb + h * o_sh + sub * 8;
    const T* gp = d_o + b * g_sb + h * g_sh + sub * 8;
    const T* lp = cp.o_lo ? reinterpret_cast<const T*>(cp.o_lo) + b * cp.l_sb + h * cp.l_sh + sub * 8 : nullptr;
    const T* qp = COPIES ? reinterpret_cast<const T*>(cp.q) + b * cp.q_sb + h * cp.q_sh + sub * 8 : nullptr;
    uint32_t m = 0u;
#pragma unroll 2
    for (int ps = 0; ps < kPasses; ++ps) {
        const int i = i0 + ps * kRowsPerPass;
        const int64_t row = bh * nq_pad + i;
        const bool in = i < Nq;
        uint4 vo = make_uint4(0, 0, 0, 0), vg = vo, vl = vo, vq = vo;
        if (in) {
            vo = *reinterpret_cast<const uint4*>(op + (int64_t)i * o_sn);
            vg = *reinterpret_cast<const uint4*>(gp + (int64_t)i * g_sn);
            if (lp) vl = *reinterpret_cast<const uint4*>(lp + (int64_t)i * cp.l_sn);
            if (COPIES) vq = *reinterpret_cast<const uint4*>(qp + (int64_t)i * cp.q_sn);
        }
        const T* eo = reinterpret_cast<const T*>(&vo);
        const T* eg = reinterpret_cast<const T*>(&vg);
        const T* el = reinterpret_cast<const T*>(&vl);
        float s = 0.f;
        // delta from the output as the forward computed it (o + o_lo) when the residual is there
#pragma unroll
        for (int e = 0; e < 8; ++e) s = fmaf(to_f32<T>(eo[e]) + to_f32<T>(el[e]), to_f32<T>(eg[e]), s);
#pragma unroll
        for (int off = LPR / 2; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
        const uint32_t m_mine = absmax16_acc(0u, vg);
        m = max(m, max(m_mine & 0xFFFFu, m_mine >> 16));
        int e_i = 0;
        if (COPIES) {
            // the row's largest |dO| (a bf16 bit pattern) over the lanes that share the row
            uint32_t mr = max(m_mine & 0xFFFFu, m_mine >> 16);
#pragma unroll
            for (int off = LPR / 2; off > 0; off >>= 1) mr = max(mr, __shfl_xor_sync(0xffffffffu, mr, off));
            e_i = log2_bound_bits(mr << 16) - 15;
            if (in) {
                const int64_t at = (((int64_t)b * Nq + i) * H + h) * D + sub * 8;
                const uint64_t mul2 = f2_pack(pow2i(-e_i), pow2i(-e_i));
                *reinterpret_cast<uint4*>(cp.q16 + at) = make_uint4(bf16x2_to_f16x2(vq.x), bf16x2_to_f16x2(vq.y),
                                                                    bf16x2_to_f16x2(vq.z), bf16x2_to_f16x2(vq.w));
                *reinterpret_cast<uint4*>(cp.do16 + at) = make_uint4(bf16x2_to_f16x2(vg.x, mul2), bf16x2_to_f16x2(vg.y, mul2),
                                                                     bf16x2_to_f16x2(vg.z, mul2), bf16x2_to_f16x2(vg.w, mul2));
            }
        }
        if (sub == 0) {
            if (in) { delta[row] = -s * pow2i(-e_i); lse2[row] = kPShift - lse[bh * Nq + i] * kLog2e + (float)e_i; }
            else    { delta[row] = 0.f; lse2[row] = -INFINITY; }
            if (COPIES) cp.erow[row] = in ? (float)e_i : 0.f;
        }
    }
    const int group = H / Hkv;
    absmax16_commit<T>(m, ranges + 2 * ((int64_t)b * Hkv + h / group), red);
}

// fused backward: fp32 dQ sums (tiles of [D/4][128 rows][4]) * scale -> dQ in the call's dtype and layout
template <typename T, int D>
__global__ void __launch_bounds__(256)
bwd_dq_convert_kernel(const float* __restrict__ acc, T* __restrict__ dq, int Nq, int H, int n_tiles, float scale_in,
                      int64_t sb, int64_t sn, int64_t sh, const float* __restrict__ ranges, int Hkv, float inv_keep) {
    const int tile = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    // the sums carry the column's dS scaling (see "number formats"): the same constant the dK epilogue uses
    const float scale = make_scales(ranges + 2 * ((int64_t)b * Hkv + h / (H / Hkv)), D, inv_keep, scale_in,
                                    kDoAsIs).acc1_mul;     // acc1_mul does not depend on dO's form
    const float* src = acc + (((int64_t)b * H + h) * n_tiles + tile) * (int64_t)(kTile * D);
    const int row = threadIdx.x & 127;
    const int i = tile * kTile + row;
    if (i >= Nq) return;
    T* out = dq + b * sb + (int64_t)i * sn + h * sh;
#pragma unroll
    for (int cg = threadIdx.x >> 7; cg < D / 8; cg += 2) {      // 8 columns = two 4-column groups
        const float4 lo = *reinterpret_cast<const float4*>(src + ((int64_t)(2 * cg) * kTile + row) * 4);
        const float4 hi = *reinterpret_cast<const float4*>(src + ((int64_t)(2 * cg + 1) * kTile + row) * 4);
        uint4 v4;
        v4.x = pack2<std::is_same<T, __nv_bfloat16>::value>(lo.x * scale, lo.y * scale);
        v4.y = pack2<std::is_same<T, __nv_bfloat16>::value>(lo.z * scale, lo.w * scale);
        v4.z = pack2<std::is_same<T, __nv_bfloat16>::value>(hi.x * scale, hi.y * scale);
        v4.w = pack2<std::is_same<T, __nv_bfloat16>::value>(hi.z * scale, hi.w * scale);
        *reinterpret_cast<uint4*>(out + cg * 8) = v4;
    }
}

// INLINE: bf16 call without room for the fp16 copies (the workspace-free entry point): the main kernels
// convert their tiles themselves.
// the kernel instance and its shared memory for a dropout form (0 none, 1 drawn in the kernel, 2 loaded;
// the converting-in-kernel instances, which serve the entry without a workspace, never load)
template <int D, bool BF16, int MODE, bool INLINE>
auto pick_kernel(int drop) {
    if (drop == 2 && !INLINE) return bwd_sm100_kernel<D, BF16, MODE, kNWG, INLINE ? 1 : 2, INLINE>;
    return drop ? bwd_sm100_kernel<D, BF16, MODE, kNWG, 1, INLINE> : bwd_sm100_kernel<D, BF16, MODE, kNWG, 0, INLINE>;
}
template <int D, int MODE>
int pick_smem(int drop) {
    return drop == 2 ? BwdCfg<D, MODE, 2>::kSmemBytes : (drop ? BwdCfg<D, MODE, 1>::kSmemBytes : BwdCfg<D, MODE, 0>::kSmemBytes);
}

template <int D, bool BF16, bool INLINE>
int launch(const fa_b200_params& p, const BwdWorkspace& ws) {
    using T = typename std::conditional<BF16, __nv_bfloat16, __half>::type;
    const CUtensorMapDataType dt = BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    constexpr bool COPIES = BF16 && !INLINE;
    cudaStream_t st = (cudaStream_t)p.stream;
    const int nq_pad = (int)align_up((size_t)p.Nq, 128);
    char* wsp = (char*)p.workspace;
    float* delta = (float*)(wsp + ws.delta_off);
    float* lse2 = (float*)(wsp + ws.lse2_off);
    float* ranges = (float*)(wsp + ws.rng_off);
    if (COPIES && (ws.q16_bytes == 0 || ws.do16_bytes == 0)) { set_error("workspace layout lacks the fp16 copies"); return FA_EWORKSPACE; }

    const bool fused = ws.dq_bytes > 0;
    float* dq_acc = fused ? (float*)(wsp + ws.dq_off) : nullptr;
    // dropout: 0 none, 1 the kernels draw their bits, 2 they load them from the call's bit buffer
    int drop = dropout_threshold(p.dropout_p) != 0u ? 1 : 0;
    const size_t bits_one = dropout_bits_bytes(p);
    if (!INLINE && drop && p.dropout_bits && p.dropout_bits_bytes >= 2 * bits_one) drop = 2;

    const int phases = p.bwd_phases ? p.bwd_phases : 7;
    if (phases & 1) {
        if (fused) FA_CUDA_CHECK(cudaMemsetAsync(dq_acc, 0, ws.dq_bytes, st));
        FA_CUDA_CHECK(cudaMemsetAsync(ranges, 0, ws.rng_bytes, st));
        const int64_t n_row_blocks64 = (int64_t)p.B * p.H * (nq_pad / 128);      // one block per 128-row tile
        const int v_slabs = (p.Nk + 255) / 256;
        const int64_t n_blocks = n_row_blocks64 + (int64_t)p.B * p.Hkv * v_slabs;
        if (n_blocks > 0x7fffffff) { set_error("problem too large for the preprocess grid"); return FA_EUNSUPPORTED; }
        const int n_row_blocks = (int)n_row_blocks64;
        PreprocessCopies cp = {};
        cp.o_lo = p.o_lo.ptr; cp.l_sb = p.o_lo.stride_b; cp.l_sn = p.o_lo.stride_n; cp.l_sh = p.o_lo.stride_h;
        if (COPIES) {
            cp.q = p.q.ptr; cp.q_sb = p.q.stride_b; cp.q_sn = p.q.stride_n; cp.q_sh = p.q.stride_h;
            cp.q16 = (uint16_t*)(wsp + ws.q16_off); cp.do16 = (uint16_t*)(wsp + ws.do16_off);
            cp.erow = (float*)(wsp + ws.erow_off);
        }
        bwd_preprocess_kernel<T, D, COPIES><<<(unsigned)n_blocks, 256, 0, st>>>(
            (const T*)p.o.ptr, (const T*)p.d_o.ptr, p.lse, lse2, delta, ranges, p.B, p.Nq, p.H, p.Hkv, nq_pad,
            p.o.stride_b, p.o.stride_n, p.o.stride_h, p.d_o.stride_b, p.d_o.stride_n, p.d_o.stride_h,
            (const T*)p.v.ptr, p.v.stride_b, p.v.stride_n, p.v.stride_h, p.Nk, p.kv_lengths, n_row_blocks, v_slabs, cp);
        FA_CUDA_CHECK(cudaGetLastError());
    }

    CUtensorMap mq, mk, mv, mg, mdq, mdk, mdv, mq16, mg16, mk16;
    int r;
    auto mk_map = [&](CUtensorMap* m, const fa_b200_tensor& t, int N, int H) {
        return cached_tmap_bnhd(m, t.ptr, dt, 2, p.B, N, H, D, t.stride_b, t.stride_n, t.stride_h, 128, 64, true);
    };
    // a dense fp16 (B, N, H, D) copy in the workspace
    auto mk_copy = [&](CUtensorMap* m, size_t off, int N, int H) {
        return cached_tmap_bnhd(m, wsp + off, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, p.B, N, H, D, (int64_t)N * H * D,
                                (int64_t)H * D, (int64_t)D, 128, 64, true);
    };
    if ((r = mk_map(&mq, p.q, p.Nq, p.H)) || (r = mk_map(&mk, p.k, p.Nk, p.Hkv)) ||
        (r = mk_map(&mv, p.v, p.Nk, p.Hkv)) || (r = mk_map(&mg, p.d_o, p.Nq, p.H)) ||
        (r = mk_map(&mdq, p.dq, p.Nq, p.H)) || (r = mk_map(&mdk, p.dk, p.Nk, p.Hkv)) ||
        (r = mk_map(&mdv, p.dv, p.Nk, p.Hkv))) {
        set_error("cuTensorMapEncodeTiled failed (%d)", r);
        return FA_ECUDA;
    }
    mq16 = mq; mg16 = mg; mk16 = mk;
    if (COPIES) {
        if ((r = mk_copy(&mq16, ws.q16_off, p.Nq, p.H)) || (r = mk_copy(&mg16, ws.do16_off, p.Nq, p.H)) ||
            (ws.k16_bytes && (r = mk_copy(&mk16, ws.k16_off, p.Nk, p.Hkv)))) {
            set_error("cuTensorMapEncodeTiled failed (%d)", r);
            return FA_ECUDA;
        }
    }
    BwdArgs a;
    a.lse2 = lse2; a.delta = delta; a.ranges = ranges; a.dq_acc = dq_acc; a.status = p.status_word; a.wait_limit_ms = p.wait_limit_ms;
    a.erow = COPIES ? (const float*)(wsp + ws.erow_off) : nullptr;
    a.kv_len = p.kv_lengths;
    a.B = p.B; a.Nq = p.Nq; a.Nk = p.Nk; a.H = p.H; a.Hkv = p.Hkv; a.nq_pad = nq_pad;
    {
        // columns whose Q, K, V and dO (16-bit) fit the budget
        const int64_t col_bytes = 2 * ((int64_t)p.Nq + p.Nk) * D * 2;
        const int64_t g = (int64_t)tile::kBwdGroupBytes / (col_bytes > 0 ? col_bytes : 1);
        a.cols_per_group = (int)(g < 1 ? 1 : (g > 65535 ? 65535 : g));
    }
    a.causal = p.causal;
    a.shift = p.causal ? p.causal_shift : 0;
    a.scale = p.scale;
    a.scale_log2 = p.scale * kLog2e;
    a.drop_thr = dropout_threshold(p.dropout_p);
    a.inv_keep = 1.f / (1.f - dropout_effective_p(p.dropout_p));
    a.key = philox_make_key(p.seed, p.offset);
    a.rng = dropout_origin_of(p);
    a.bits_q = (const uint4*)p.dropout_bits;
    a.bits_k = (const uint32_t*)((const char*)p.dropout_bits + bits_one);
    a.nk_pad = (int)align_up((size_t)p.Nk, 128);
    if (drop == 2 && !p.dropout_bits_ready && (phases & 1)) {
        int rc = launch_dropout_bits(p, (void*)a.bits_q, (void*)a.bits_k);
        if (rc) return rc;
    }

    static std::mutex smem_mu;             // per (D, dtype, INLINE) instance of this function
    static uint64_t smem_done[9] = {};     // [kernel mode x dropout form] -> devices whose limit is set
    constexpr int kThreads = 128 * kNWG + kExtraThreads;
    const dim3 grid_kv((p.Nk + kTile - 1) / kTile, p.Hkv, p.B);
    const dim3 grid_q((p.Nq + kTile - 1) / kTile, p.H, p.B);
    if constexpr (D == 64) if (fused) {
        // one key-stationary kernel for dK, dV and the fp32 dQ sums, then the conversion of dQ
        auto k2 = pick_kernel<D, BF16, 2, INLINE>(drop);
        const int smem2 = pick_smem<D, 2>(drop);
        FA_CUDA_CHECK(set_smem_limit_once(k2, smem2, p.device, &smem_done[6 + drop], &smem_mu));
        if (phases & 2) {
            k2<<<grid_kv, kThreads, smem2, st>>>(mk, mv, mq16, mg16, mdk, mdv, mdk, a);
            FA_CUDA_CHECK(cudaGetLastError());
        }
        if (phases & 4) {
            bwd_dq_convert_kernel<T, D><<<grid_q, 256, 0, st>>>(dq_acc, (T*)p.dq.ptr, p.Nq, p.H, nq_pad / kTile, p.scale,
                                                               p.dq.stride_b, p.dq.stride_n, p.dq.stride_h, ranges, p.Hkv,
                                                               a.inv_keep);
            FA_CUDA_CHECK(cudaGetLastError());
        }
        return FA_OK;
    }
    if (COPIES && ws.k16_bytes == 0) { set_error("workspace layout lacks the fp16 copy of K"); return FA_EWORKSPACE; }
    auto k0 = pick_kernel<D, BF16, 0, INLINE>(drop);
    auto k1 = pick_kernel<D, BF16, 1, INLINE>(drop);
    const int smem0 = pick_smem<D, 0>(drop), smem1 = pick_smem<D, 1>(drop);
    FA_CUDA_CHECK(set_smem_limit_once(k0, smem0, p.device, &smem_done[drop], &smem_mu));
    FA_CUDA_CHECK(set_smem_limit_once(k1, smem1, p.device, &smem_done[3 + drop], &smem_mu));
    if (phases & 2) {
        // stationary K_j, V_j; streamed Q_i, dO_i (bf16 with copies: their fp16 copies; the kernel leaves
        // the fp16 copy of K behind for the dQ kernel)
        k0<<<grid_kv, kThreads, smem0, st>>>(mk, mv, mq16, mg16, mdk, mdv, mk16, a);
        FA_CUDA_CHECK(cudaGetLastError());
    }
    if (phases & 4) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = grid_q; cfg.blockDim = dim3(kThreads); cfg.dynamicSmemBytes = smem1; cfg.stream = st;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        // Only behind the dK/dV kernel of this call, and only while one head's K and V are small
        // beside L2 (the two kernels stream different heads' tiles at the same time): measured on
        // B200 (H32 D128 causal) the overlap takes 1 % off the backward at N = 4096; longer
        // sequences showed no gain.  Never with the fp16 copies: the dQ kernel streams the copy of K
        // that the dK/dV kernel is still writing.
        cfg.numAttrs = (!COPIES && (phases & 2) && (int64_t)p.Nk * D * 4 <= (int64_t)tile::kBwdOverlapMaxKvBytes) ? 1 : 0;
        // stationary Q_i (its fp16 copy), dO_i; streamed K_j (its fp16 copy), V_j
        FA_CUDA_CHECK(cudaLaunchKernelEx(&cfg, k1, mq16, mg, mk16, mv, mdq, mdq, mdq, a));
    }
    return FA_OK;
}

}  // namespace

bool sm100_bwd_fused_supported(const fa_b200_params& p) {
    // D = 64 only.  At D = 128 tensor memory is full (S^T, dP^T, dK, dV), the per-step dQ tile has
    // to share dP^T's columns, which serialises the step, and the fp32 additions (64 KB per step)
    // cost more than recomputing S and dP in a second kernel: measured on B200 (B4 N4096 H32
    // causal) 2.12 ms against 1.95 ms for the two kernels.
    return tile::bwd_one_kernel(p.D);
}

int sm100_bwd(const fa_b200_params& p, const BwdWorkspace& ws) {
    if (p.dtype == FA_B200_BF16) {
        if (ws.q16_bytes == 0) return p.D == 128 ? launch<128, true, true>(p, ws) : launch<64, true, true>(p, ws);
        return p.D == 128 ? launch<128, true, false>(p, ws) : launch<64, true, false>(p, ws);
    }
    return p.D == 128 ? launch<128, false, false>(p, ws) : launch<64, false, false>(p, ws);
}

}  // namespace fa
