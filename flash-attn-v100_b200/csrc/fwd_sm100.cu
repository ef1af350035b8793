// Attention forward for sm_100a: TMA -> shared memory -> tcgen05.mma with
// accumulators in tensor memory, warp-specialised, persistent.
//
// Replaces the reference's Triton forward kernel
// (kernels/forward_kernel.py:18-243) and its launcher (:246-387).
//
// Work: a "pair" is two consecutive 128-row query tiles of one (batch, head);
// it walks the key/value sequence in 128-row blocks.  The grid is one CTA per
// SM; CTA c processes work items c, c + grid, c + 2 grid, ...  Under a causal
// mask an item is a pair together with its mirror (pair p and pair P-1-p), so
// that every item costs the same number of key blocks and a static round-robin
// is balanced; items of one head are adjacent, so the CTAs running at any time
// share a few heads' K/V in L2.  Nothing is re-initialised between pairs: the
// K/V ring, the barriers' phases and tensor memory carry on, and the next
// pair's Q and first K/V blocks are loaded while the current pair drains.
//
//   warp 9      TMA producer: Q tiles per pair, K_j / V_j into two rings
//   warp 8      MMA issuer (one elected thread):
//                   S_t = Q_t K_j^T          (SS MMA, both operands K-major)
//                   O_t += P_t V_j           (TS MMA: P_t from TMEM, V_j MN-major)
//               issue order  S0(0) S1(0) | PV0(j) S0(j+1) PV1(j) S1(j+1) ...
//               so that the softmax of one tile overlaps the MMAs of the other; each PV
//               is issued in two 64-key halves, the first as soon as that half of P_t
//               is in TMEM (the threads are still computing the second)
//   warps 0-3   softmax + epilogue of tile 0, one thread per query row (TMEM lane)
//   warps 4-7   softmax + epilogue of tile 1
//   warps 10-11 bf16 inputs: convert each V_j tile to fp16 in place as it lands, so that PV runs
//               f16 x f16 with P rounded to fp16 instead of bf16 (see sm100_ptx.cuh); fp16 inputs: idle
//               (the two warps complete the third warpgroup for setmaxnreg)
//
// Online softmax in the log2 domain with scale*log2(e) folded into one FMA.
// The running maximum is only refreshed when it grows by more than 2^8 (warp
// vote), so the O accumulator in TMEM is rescaled rarely; the final division
// by the row sum makes the result exact either way.  P is rounded to fp16 (whatever
// the input dtype) and written over S in TMEM; dropout zeroes P entries (the 1/(1-p)
// factor is applied once to O), the row sum uses the undropped P.
//
// TMEM columns: S0/P0 [0,128)  S1/P1 [128,256)  O0 [256,256+D)  O1 [384,384+D).
// O_t of the next pair is first written by a PV MMA that waits for P_t, which
// the owning threads produce only after their epilogue has read O_t.
//
// Every mbarrier wait is bounded; on a time-out the CTA raises its abort flag,
// every role unwinds, TMEM is freed and the status word is set.
#include "fa_common.cuh"
#include "sm100_ptx.cuh"
#include "tma_host.cuh"
#include "tile_config.cuh"
#include <type_traits>

namespace fa {
namespace {

using namespace ptx;

constexpr int kBlockM = tile::kBlockM;      // query rows per tile
constexpr int kBlockN = tile::kBlockN;      // key rows per block
constexpr int kThreads = 32 * tile::kFwdWarps;   // 2 softmax warpgroups + 1 warpgroup holding the MMA, TMA and converting warps
constexpr int kBoxBytes = 128 * 128;   // one TMA box: 128 rows x 64 16-bit elements
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr float kRescaleThreshold = tile::kFwdRescaleLog2;   // log2 units
// Share of the exponentials evaluated by the FMA-pipe polynomial instead of the special-function
// unit: in kPolyCount of every kPolyPeriod groups of four, two (tile_config.cuh has the measurements).
constexpr int kPolyPeriod = tile::kFwdPolyPeriod, kPolyCount = tile::kFwdPolyCount;
// The first 64 keys of P are handed to the MMA warp after this many of the second half's 64
// exponentials (a multiple of 4), when their tcgen05.st has had time to complete.
constexpr int kHalfSignalAt = tile::kFwdHalfSignalAt;
// Register split after setmaxnreg.  The pool is what the CTA was launched with, 168 registers for
// each of its 384 threads, not the whole file: a split that asks for more makes
// setmaxnreg.inc wait for ever.
constexpr int kRegsSoftmax = tile::kFwdRegsSoftmax, kRegsOther = tile::kFwdRegsOther;
static_assert(256 * kRegsSoftmax + 128 * kRegsOther <= 168 * kThreads, "register split exceeds the CTA's allocation");
static_assert(tile::kFwdQTilesPerCta == 2, "the kernel is written for two query tiles per work item");

template <int D>
struct FwdCfg {
    static constexpr int kNBox = D / 64;
    static constexpr int kTileBytes = kNBox * kBoxBytes;
    static constexpr int kStages = tile::fwd_kv_stages(D);
    // barrier slots
    static constexpr int kQFull = 0;                       // [2]
    static constexpr int kQEmpty = 2;                      // [2] last S MMA of the pair has read Q_t
    static constexpr int kKFull = 4;                       // [kStages]
    static constexpr int kKEmpty = kKFull + kStages;
    static constexpr int kVFull = kKEmpty + kStages;
    static constexpr int kVEmpty = kVFull + kStages;
    static constexpr int kSFull = kVEmpty + kStages;       // [2]
    static constexpr int kPFull = kSFull + 2;              // [2] one arrival per warp of the warpgroup
    static constexpr int kODone = kPFull + 2;              // [2]
    static constexpr int kPHalf = kODone + 2;              // [2] first 64 keys of P_t stored (one arrival per warp)
    static constexpr int kVConv = kPHalf + 2;              // [kStages] V_j converted to fp16 (one arrival per converting warp)
    static constexpr int kNumBars = kVConv + kStages;
    static constexpr int kSmemBytes = (2 + 2 * kStages) * kTileBytes + kNumBars * 8 + 64 + 1024;
};

struct FwdArgs {
    void* o;                       // (B, Nq, H, D) output, element strides below
    int64_t o_sb, o_sn, o_sh;
    void* o_lo;                    // optional residual of the output (what rounding O to 16 bits dropped)
    int64_t l_sb, l_sn, l_sh;
    float* lse;
    int32_t* status;
    const int32_t* kv_len;         // optional per-batch key counts
    int B, Nq, Nk, H, Hkv;
    int causal;
    int shift;                     // key j is visible to query i iff j <= i + shift
    int n_pairs;                   // ceil(Nq / 256)
    int items_per_head;            // causal: ceil(n_pairs / 2) mirrored items; else n_pairs
    int n_items;                   // items_per_head * B * H
    int wait_limit_ms;             // limit of one mbarrier wait (0: the default)
    float scale_log2;              // scale * log2(e)
    uint32_t drop_thr;
    float inv_keep;
    PhiloxKey key;
    DropoutOrigin rng;
    const uint4* mq;               // DROP = 2: keep bits, [(b*H + h) * n_kblocks + key block][padded query row]
    int nq_pad, n_kblocks;
};

struct Pair { int pair, h, b; };

// Sub-item u (0 or 1) of work item w; false if the item has no such sub-item.
__device__ __forceinline__ bool decode_work(const FwdArgs& a, int w, int u, Pair& out) {
    const int bh = w / a.items_per_head, slot = w - bh * a.items_per_head;
    int pair;
    if (a.causal) {
        const int heavy = a.n_pairs - 1 - slot;           // more key blocks: first
        if (u == 0) pair = heavy;
        else { if (slot == heavy) return false; pair = slot; }
    } else {
        if (u == 1) return false;
        pair = slot;
    }
    out.pair = pair;
    out.h = bh % a.H;
    out.b = bh / a.H;
    return true;
}

// key blocks tile t of a pair visits
__device__ __forceinline__ int num_blocks(const FwdArgs& a, int pair, int t, int nk) {
    const int row0 = (pair * 2 + t) * kBlockM;
    int kv_end = nk;               // keys this batch entry attends to
    if (a.causal && row0 + kBlockM + a.shift < kv_end) kv_end = row0 + kBlockM + a.shift;
    return (row0 < a.Nq) ? (kv_end + kBlockN - 1) / kBlockN : 0;
}

// P is stored as 2^(S c - m + kPShift): with the lazily refreshed maximum P <= 2^8, so the shifted value
// stays below 2^14 in fp16 and entries down to 2^-20 of the row's largest keep full precision.
constexpr float kPShift = 6.0f;

// DROP: 0 no dropout; 1 the keep bits are drawn here, by the softmax threads (no workspace);
// 2 they are loaded from the workspace, where dropout_bits_kernel has written the call's bits.
template <int D, bool BF16, int DROP>
__global__ void __launch_bounds__(kThreads, 1)
fwd_sm100_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                 const __grid_constant__ CUtensorMap map_v, const FwdArgs a) {
    using Cfg = FwdCfg<D>;
    constexpr int ST = Cfg::kStages;
    constexpr int TILE = Cfg::kTileBytes;
    // tcgen05.mma kind::f16 wants A and B in one format (an fp16 A next to a bf16 B raises an
    // illegal-instruction fault).  P is always fp16; a bf16 V tile is converted to fp16 in shared memory.
    constexpr bool CONV = BF16;
    constexpr bool P_BF16 = false;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* sQ = smem;
    uint8_t* sK = sQ + 2 * TILE;
    uint8_t* sV = sK + ST * TILE;
    uint64_t* bars = (uint64_t*)(sV + ST * TILE);
    uint32_t* tmem_slot = (uint32_t*)(bars + Cfg::kNumBars);
    volatile uint32_t* abort_flag = (volatile uint32_t*)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int group = a.H / a.Hkv;

    if (threadIdx.x == 0) {
        for (int i = 0; i < Cfg::kNumBars; ++i) {
            const bool wg_bar = (i >= Cfg::kPFull && i < Cfg::kPFull + 2) || (i >= Cfg::kPHalf && i < Cfg::kPHalf + 2);
            const bool conv_bar = (i >= Cfg::kVConv && i < Cfg::kVConv + ST);
            mbar_init(&bars[i], wg_bar ? 4u : (conv_bar ? 2u : 1u));
        }
        wait_control_init(abort_flag, a.wait_limit_ms);
        fence_mbar_init();
    }
    if (warp == 8) {
        tmem_alloc(tmem_slot, 512);
        tmem_relinquish();
    }
    if (warp == 9 && lane == 0) {
        prefetch_tensormap(&map_q);
        prefetch_tensormap(&map_k);
        prefetch_tensormap(&map_v);
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;

    if (warp >= 8) {
      asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsOther));
      if (warp == 9) {
        // ------------------------------------------------------------ TMA producer
        if (elect_one()) {
            int kvc = 0;                    // K/V blocks loaded so far (ring index = count % ST)
            int q_loads[2] = {0, 0};
            bool ok = true;
            for (int w = blockIdx.x; w < a.n_items && ok; w += gridDim.x) {
                for (int u = 0; u < 2 && ok; ++u) {
                    Pair pr;
                    if (!decode_work(a, w, u, pr)) continue;
                    const int hk = pr.h / group;
                    const int q0 = pr.pair * 2 * kBlockM;
                    const int nk = kv_len_of(a.kv_len, pr.b, a.Nk);
                    const int n0 = num_blocks(a, pr.pair, 0, nk), n1 = num_blocks(a, pr.pair, 1, nk);
                    const int nmax = n0 > n1 ? n0 : n1;
#pragma unroll
                    for (int t = 0; t < 2; ++t) {
                        if ((t == 0 ? n0 : n1) == 0) continue;
                        // Q_t of the previous pair must have been read by its last S MMA
                        ok = mbar_wait(&bars[Cfg::kQEmpty + t], ((uint32_t)q_loads[t] & 1u) ^ 1u, abort_flag);
                        if (!ok) break;
                        mbar_expect_tx(&bars[Cfg::kQFull + t], TILE);
#pragma unroll
                        for (int bx = 0; bx < Cfg::kNBox; ++bx)
                            tma_load_4d(sQ + t * TILE + bx * kBoxBytes, &map_q, &bars[Cfg::kQFull + t],
                                        bx * 64, pr.h, q0 + t * kBlockM, pr.b);
                        ++q_loads[t];
                    }
                    for (int j = 0; j < nmax && ok; ++j, ++kvc) {
                        const int s = kvc % ST;
                        const uint32_t ph = (uint32_t)(kvc / ST) & 1u;
                        ok = mbar_wait(&bars[Cfg::kKEmpty + s], ph ^ 1u, abort_flag);
                        if (!ok) break;
                        mbar_expect_tx(&bars[Cfg::kKFull + s], TILE);
#pragma unroll
                        for (int bx = 0; bx < Cfg::kNBox; ++bx)
                            tma_load_4d(sK + s * TILE + bx * kBoxBytes, &map_k, &bars[Cfg::kKFull + s],
                                        bx * 64, hk, j * kBlockN, pr.b);
                        ok = mbar_wait(&bars[Cfg::kVEmpty + s], ph ^ 1u, abort_flag);
                        if (!ok) {
                            // K of this block is in flight: let it land before giving up shared memory
                            for (int spin = 0; spin < 4096 && !mbar_try_wait(&bars[Cfg::kKFull + s], ph); ++spin) {}
                            break;
                        }
                        mbar_expect_tx(&bars[Cfg::kVFull + s], TILE);
#pragma unroll
                        for (int bx = 0; bx < Cfg::kNBox; ++bx)
                            tma_load_4d(sV + s * TILE + bx * kBoxBytes, &map_v, &bars[Cfg::kVFull + s],
                                        bx * 64, hk, j * kBlockN, pr.b);
                    }
                }
            }
            if (!ok) {
                // unwinding: let copies already issued land before the CTA gives up its
                // shared memory (bounded: a copy that has not landed by now never will)
                for (int s = 0; s < ST; ++s) {
                    const int nf = (kvc + ST - 1 - s) / ST;       // completed K+V fills of stage s
                    for (int spin = 0; spin < 4096 && nf > 0 &&
                         !mbar_try_wait(&bars[Cfg::kKFull + s], (uint32_t)(nf - 1) & 1u); ++spin) {}
                    for (int spin = 0; spin < 4096 && nf > 0 &&
                         !mbar_try_wait(&bars[Cfg::kVFull + s], (uint32_t)(nf - 1) & 1u); ++spin) {}
                }
                for (int t = 0; t < 2; ++t)
                    for (int spin = 0; spin < 4096 && q_loads[t] > 0 &&
                         !mbar_try_wait(&bars[Cfg::kQFull + t], (uint32_t)(q_loads[t] - 1) & 1u); ++spin) {}
            }
        }
        __syncwarp();
      } else if (warp == 8) {
        // ------------------------------------------------------------ MMA issuer
        if (elect_one()) {
            constexpr uint32_t idesc_s = make_idesc_f16(BF16, BF16, kBlockM, kBlockN, false, false);
            constexpr uint32_t idesc_pv = make_idesc_f16(false, false, kBlockM, D, false, true);   // P, V: fp16
            const uint32_t sQ_u = smem_u32(sQ), sK_u = smem_u32(sK), sV_u = smem_u32(sV);

            // Descriptors differ only in the 16-byte-granular start address held in their low
            // bits: build one per buffer here and add offsets in the issue loops, which keeps the
            // single issuing thread's instruction count per MMA small.
            const uint64_t dQ = make_smem_desc_sw128(sQ_u, 0, 1024);
            const uint64_t dK = make_smem_desc_sw128(sK_u, 0, 1024);
            const uint64_t dV = make_smem_desc_sw128(sV_u, kBoxBytes, 1024);
            auto issue_s = [&](int t, int ks) {
                const uint64_t a0 = dQ + (uint64_t)((t * TILE) >> 4), b0 = dK + (uint64_t)((ks * TILE) >> 4);
                const uint32_t d = tmem + (uint32_t)t * 128u;
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const uint32_t off = ((uint32_t)(kk >> 2) * kBoxBytes + (uint32_t)(kk & 3) * 32u) >> 4;
                    mma_ss_f16(d, a0 + off, b0 + off, idesc_s, kk > 0);
                }
            };
            // one 64-key half (hf = 0, 1) of O_t += P_t V_j
            auto issue_pv = [&](int t, int vs, bool acc, int hf) {
                const uint64_t b0 = dV + (uint64_t)((vs * TILE) >> 4);
                const uint32_t d = tmem + 256u + (uint32_t)t * 128u, a0 = tmem + (uint32_t)t * 128u;
#pragma unroll
                for (int k4 = 0; k4 < kBlockN / 32; ++k4) {
                    const int kk = hf * (kBlockN / 32) + k4;
                    mma_ts_f16(d, a0 + (uint32_t)kk * 8u, b0 + (uint64_t)((kk * 2048) >> 4), idesc_pv,
                               (acc || kk > 0) ? 1u : 0u);
                }
            };

            int kvc = 0;                    // K/V blocks consumed so far
            int q_uses[2] = {0, 0};         // pairs that used tile t (Q_full phase)
            int p_waits[2] = {0, 0};        // P_t hand-offs so far (P_full phase)
            bool ok = true;
            for (int w = blockIdx.x; w < a.n_items && ok; w += gridDim.x) {
                for (int u = 0; u < 2 && ok; ++u) {
                    Pair pr;
                    if (!decode_work(a, w, u, pr)) continue;
                    const int nk = kv_len_of(a.kv_len, pr.b, a.Nk);
                    int nblk[2] = {num_blocks(a, pr.pair, 0, nk), num_blocks(a, pr.pair, 1, nk)};
                    const int nmax = nblk[0] > nblk[1] ? nblk[0] : nblk[1];
#pragma unroll
                    for (int t = 0; t < 2; ++t) {
                        if (nblk[t] == 0) continue;
                        if (ok) ok = mbar_wait(&bars[Cfg::kQFull + t], (uint32_t)q_uses[t] & 1u, abort_flag);
                        ++q_uses[t];
                    }
                    if (ok) ok = mbar_wait(&bars[Cfg::kKFull + kvc % ST], (uint32_t)(kvc / ST) & 1u, abort_flag);
                    if (!ok) break;
                    tc_fence_after_sync();
#pragma unroll
                    for (int t = 0; t < 2; ++t) {
                        if (nblk[t] == 0) continue;
                        issue_s(t, kvc % ST);
                        mma_commit(&bars[Cfg::kSFull + t]);
                        if (nblk[t] == 1) mma_commit(&bars[Cfg::kQEmpty + t]);
                    }
                    mma_commit(&bars[Cfg::kKEmpty + kvc % ST]);

                    for (int j = 0; j < nmax && ok; ++j) {
                        const int vs = (kvc + j) % ST;
                        const uint32_t vph = (uint32_t)((kvc + j) / ST) & 1u;
                        const int ks = (kvc + j + 1) % ST;
                        const uint32_t kph = (uint32_t)((kvc + j + 1) / ST) & 1u;
                        bool k_ready = false;
                        ok = mbar_wait(&bars[(CONV ? Cfg::kVConv : Cfg::kVFull) + vs], vph, abort_flag);
                        if (!ok) break;
#pragma unroll
                        for (int t = 0; t < 2; ++t) {
                            if (j < nblk[t]) {
                                // the first 64 keys of P_t arrive while the second 64 are still computed
                                ok = mbar_wait(&bars[Cfg::kPHalf + t], (uint32_t)p_waits[t] & 1u, abort_flag);
                                if (!ok) break;
                                tc_fence_after_sync();
                                issue_pv(t, vs, j > 0, 0);
                                ok = mbar_wait(&bars[Cfg::kPFull + t], (uint32_t)p_waits[t] & 1u, abort_flag);
                                if (!ok) break;
                                ++p_waits[t];
                                tc_fence_after_sync();
                                issue_pv(t, vs, j > 0, 1);
                                if (j == nblk[t] - 1) mma_commit(&bars[Cfg::kODone + t]);
                            }
                            if (t == 1) mma_commit(&bars[Cfg::kVEmpty + vs]);
                            if (j + 1 < nblk[t]) {
                                if (!k_ready) {
                                    ok = mbar_wait(&bars[Cfg::kKFull + ks], kph, abort_flag);
                                    if (!ok) break;
                                    k_ready = true;
                                    tc_fence_after_sync();
                                }
                                issue_s(t, ks);
                                mma_commit(&bars[Cfg::kSFull + t]);
                                if (j + 2 == nblk[t]) mma_commit(&bars[Cfg::kQEmpty + t]);   // last S of tile t
                            }
                        }
                        if (ok && j + 1 < nmax) mma_commit(&bars[Cfg::kKEmpty + ks]);
                    }
                    kvc += nmax;
                }
            }
        }
        __syncwarp();
      } else if (CONV) {
        // ------------------------------------------------------------ warps 10-11: V_j bf16 -> fp16
        // the same walk as the producer's; a tile is touched between its arrival (V_full) and its
        // first reader (the PV MMAs wait for V_conv instead of V_full)
        const int ct = (warp - 10) * 32 + lane;
        int kvc = 0;
        bool ok = true;
        for (int w = blockIdx.x; w < a.n_items && ok; w += gridDim.x) {
            for (int u = 0; u < 2 && ok; ++u) {
                Pair pr;
                if (!decode_work(a, w, u, pr)) continue;
                const int nk = kv_len_of(a.kv_len, pr.b, a.Nk);
                const int n0 = num_blocks(a, pr.pair, 0, nk), n1 = num_blocks(a, pr.pair, 1, nk);
                const int nmax = n0 > n1 ? n0 : n1;
                for (int j = 0; j < nmax; ++j, ++kvc) {
                    const int sidx = kvc % ST;
                    ok = mbar_wait(&bars[Cfg::kVFull + sidx], (uint32_t)(kvc / ST) & 1u, abort_flag);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    convert_tile_bf16_to_f16<false>(sV + sidx * TILE, TILE, ct, 64, 1.f);
                    fence_proxy_async_smem();           // generic-proxy writes -> visible to the MMA's reads
                    mbar_arrive_warp(&bars[Cfg::kVConv + sidx]);
                }
            }
        }
      }   // fp16 inputs: warps 10-11 idle, they complete the third warpgroup
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsSoftmax));
        // ------------------------------------------------------------ softmax + epilogue
        using T16 = typename std::conditional<BF16, __nv_bfloat16, __half>::type;
        const int t = warp >> 2;
        const int r = (warp & 3) * 32 + lane;
        const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
        const uint32_t tS = tmem + (uint32_t)t * 128u + lane_off;
        const uint32_t tO = tmem + 256u + (uint32_t)t * 128u + lane_off;
        int s_waits = 0;                 // S_t hand-offs so far (S_full phase)
        int o_waits = 0;                 // pairs finished so far (O_done phase)
        bool ok = true;

        for (int w = blockIdx.x; w < a.n_items && ok; w += gridDim.x) {
            for (int u = 0; u < 2 && ok; ++u) {
                Pair pr;
                if (!decode_work(a, w, u, pr)) continue;
                const int nk = kv_len_of(a.kv_len, pr.b, a.Nk);
                const int n = num_blocks(a, pr.pair, t, nk);
                if (n == 0) continue;
                const int tile = pr.pair * 2 + t;
                const int i = tile * kBlockM + r;                    // global query row
                const uint32_t bh = dropout_column(a.rng, pr.b, pr.h);
                float m = -INFINITY, l = 0.f;

                for (int j = 0; j < n; ++j) {
                    // DROP = 2: the block's 128 keep bits of my row, asked for before the wait for S
                    uint4 kb4 = make_uint4(0u, 0u, 0u, 0u);
                    if constexpr (DROP == 2)
                        kb4 = a.mq[((int64_t)(pr.b * a.H + pr.h) * a.n_kblocks + j) * a.nq_pad + i];
                    ok = mbar_wait(&bars[Cfg::kSFull + t], (uint32_t)s_waits & 1u, abort_flag);
                    ok = __all_sync(0xffffffffu, ok);      // the TMEM accesses below are warp-collective
                    if (!ok) break;
                    ++s_waits;
                    tc_fence_after_sync();
                    uint32_t sr[4][32];                    // the row's 128 scores, then its 128 probabilities
#define SF(c) __uint_as_float(sr[(c) >> 5][(c) & 31])
#define SSET(c, x) sr[(c) >> 5][(c) & 31] = __float_as_uint(x)
#pragma unroll
                    for (int c = 0; c < 4; ++c) tmem_ld_32x32(tS + c * 32, sr[c]);
                    tmem_wait_ld();

                    const int col0 = j * kBlockN;
                    const bool need_mask = (a.causal && col0 + kBlockN - 1 > tile * kBlockM + a.shift) || (col0 + kBlockN > nk);
                    if (need_mask) {
                        // my row sees the block's first `seen` columns: keys below the count, at most i + shift
                        int seen = nk - col0;
                        if (a.causal && i + a.shift + 1 - col0 < seen) seen = i + a.shift + 1 - col0;
#pragma unroll
                        for (int c = 0; c < 128; ++c)
                            if (c >= seen) SSET(c, -INFINITY);
                    }
                    float mx0 = SF(0), mx1 = SF(1), mx2 = SF(2), mx3 = SF(3);
#pragma unroll
                    for (int c = 4; c < 128; c += 8) {          // 3-input max: one instruction per two scores
                        mx0 = max3(mx0, SF(c), SF(c + 1)); mx1 = max3(mx1, SF(c + 2), SF(c + 3));
                        if (c + 4 < 128) { mx2 = max3(mx2, SF(c + 4), SF(c + 5)); mx3 = max3(mx3, SF(c + 6), SF(c + 7)); }
                    }
                    const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * a.scale_log2;
                    const float m_new = fmaxf(m, mx);
                    const bool grow = (m_new - m) > kRescaleThreshold;   // first block: inf > 8
                    if (__any_sync(0xffffffffu, grow)) {
                        const float alpha = ex2(m - m_new);               // 0 on the first block
                        m = m_new;
                        l *= alpha;
                        if (j > 0) {
                            // S_t(j) complete implies PV_t(j-1) complete (same issuing thread, in order)
#pragma unroll
                            for (int c0 = 0; c0 < D; c0 += 32) {
                                uint32_t orr[32];
                                tmem_ld_32x32(tO + c0, orr);
                                tmem_wait_ld();
#pragma unroll
                                for (int c = 0; c < 32; ++c) orr[c] = __float_as_uint(__uint_as_float(orr[c]) * alpha);
                                tmem_st_32x32(tO + c0, orr);
                            }
                        }
                    }
                    // P = 2^(S*c - m): packed FMAs; of every four probabilities two take the
                    // special-function unit and two either that unit or the polynomial on the FMA pipes.  Without
                    // dropout P is packed to 16 bits as it is produced and each 64-key half is
                    // stored to TMEM as soon as it is complete, so conversion and store latency
                    // overlap the exponentials of the other half.
                    const uint64_t c2 = f2_pack(a.scale_log2, a.scale_log2), nm2 = f2_pack(kPShift - m, kPShift - m);
                    uint64_t la = 0ull, lb = 0ull;             // {0.f, 0.f}
#pragma unroll
                    for (int c0 = 0; c0 < 2; ++c0) {
                        uint32_t pk[32];
#pragma unroll
                        for (int cc = 0; cc < 64; cc += 4) {
                            const int c = c0 * 64 + cc;
                            float x0, x1, x2, x3, p0, p1, p2, p3;
                            if (DROP != 1 && c0 == 1 && cc == kHalfSignalAt) {
                                // the first half's store has had these groups' time to complete
                                tmem_wait_st();
                                tc_fence_before_sync();
                                mbar_arrive_warp(&bars[Cfg::kPHalf + t]);
                            }
                            f2_unpack(f2_fma(f2_pack(SF(c), SF(c + 1)), c2, nm2), x0, x1);
                            f2_unpack(f2_fma(f2_pack(SF(c + 2), SF(c + 3)), c2, nm2), x2, x3);
                            p0 = ex2(x0); p1 = ex2(x1);
                            if (((cc >> 2) % kPolyPeriod) < kPolyCount) ex2_poly2(x2, x3, p2, p3);
                            else { p2 = ex2(x2); p3 = ex2(x3); }
                            la = f2_add(la, f2_pack(p0, p1));
                            lb = f2_add(lb, f2_pack(p2, p3));
                            if constexpr (DROP == 1) {
                                SSET(c, p0); SSET(c + 1, p1); SSET(c + 2, p2); SSET(c + 3, p3);
                            } else {
                                if constexpr (DROP == 2) {
                                    // dropped entries leave the MMA's operand, not the row sum above
                                    const uint32_t word = (c >> 5) == 0 ? kb4.x : ((c >> 5) == 1 ? kb4.y : ((c >> 5) == 2 ? kb4.z : kb4.w));
                                    const uint32_t kw = word >> (c & 31);
                                    if (!(kw & 1u)) p0 = 0.f;
                                    if (!(kw & 2u)) p1 = 0.f;
                                    if (!(kw & 4u)) p2 = 0.f;
                                    if (!(kw & 8u)) p3 = 0.f;
                                }
                                pk[cc / 2] = pack2<P_BF16>(p0, p1);
                                pk[cc / 2 + 1] = pack2<P_BF16>(p2, p3);
                            }
                        }
                        if constexpr (DROP != 1) tmem_st_32x32(tS + c0 * 32, pk);
                    }
                    {
                        float s0, s1, s2, s3;
                        f2_unpack(la, s0, s1); f2_unpack(lb, s2, s3);
                        l += (s0 + s1) + (s2 + s3);
                    }
                    if constexpr (DROP == 1) {
#pragma unroll
                        for (int g = 0; g < 8; ++g) {
                            const uint32_t bits = dropout_keep_bits(a.key, bh, (uint32_t)i, (uint32_t)(j * 8 + g), a.drop_thr);
#pragma unroll
                            for (int c = 0; c < 16; ++c)
                                if (!((bits >> c) & 1u)) SSET(g * 16 + c, 0.f);
                        }
#pragma unroll
                        for (int c0 = 0; c0 < 2; ++c0) {
                            uint32_t pk[32];
#pragma unroll
                            for (int c = 0; c < 32; ++c) pk[c] = pack2<P_BF16>(SF(c0 * 64 + 2 * c), SF(c0 * 64 + 2 * c + 1));
                            tmem_st_32x32(tS + c0 * 32, pk);
                        }
                    }
#undef SF
#undef SSET
                    tmem_wait_st();
                    tc_fence_before_sync();
                    if (DROP == 1) mbar_arrive_warp(&bars[Cfg::kPHalf + t]);
                    mbar_arrive_warp(&bars[Cfg::kPFull + t]);
                }
                if (!ok) break;

                // ---- epilogue: O_t / l -> 16 bit -> global, straight from registers
                ok = mbar_wait(&bars[Cfg::kODone + t], (uint32_t)o_waits & 1u, abort_flag);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                ++o_waits;
                tc_fence_after_sync();
                const float inv = a.inv_keep / l;
                T16* orow = reinterpret_cast<T16*>(a.o) + (int64_t)pr.b * a.o_sb + (int64_t)i * a.o_sn +
                            (int64_t)pr.h * a.o_sh;
                T16* lrow = a.o_lo ? reinterpret_cast<T16*>(a.o_lo) + (int64_t)pr.b * a.l_sb + (int64_t)i * a.l_sn +
                                         (int64_t)pr.h * a.l_sh : nullptr;
#pragma unroll
                for (int c0 = 0; c0 < D; c0 += 32) {
                    uint32_t orr[32];
                    tmem_ld_32x32(tO + c0, orr);
                    tmem_wait_ld();
                    if (i < a.Nq) {
#pragma unroll
                        for (int g = 0; g < 4; ++g) {
                            uint4 v4;
                            v4.x = pack2<BF16>(__uint_as_float(orr[g * 8 + 0]) * inv, __uint_as_float(orr[g * 8 + 1]) * inv);
                            v4.y = pack2<BF16>(__uint_as_float(orr[g * 8 + 2]) * inv, __uint_as_float(orr[g * 8 + 3]) * inv);
                            v4.z = pack2<BF16>(__uint_as_float(orr[g * 8 + 4]) * inv, __uint_as_float(orr[g * 8 + 5]) * inv);
                            v4.w = pack2<BF16>(__uint_as_float(orr[g * 8 + 6]) * inv, __uint_as_float(orr[g * 8 + 7]) * inv);
                            *reinterpret_cast<uint4*>(orow + c0 + g * 8) = v4;
                            if (lrow) {
                                // residual: the exact value minus what was just stored, rounded once more
                                const uint32_t hi[4] = {v4.x, v4.y, v4.z, v4.w};
                                uint32_t lo[4];
#pragma unroll
                                for (int e = 0; e < 4; ++e) {
                                    float h0, h1;
                                    unpack2<BF16>(hi[e], h0, h1);
                                    lo[e] = pack2<BF16>(__uint_as_float(orr[g * 8 + 2 * e]) * inv - h0,
                                                        __uint_as_float(orr[g * 8 + 2 * e + 1]) * inv - h1);
                                }
                                *reinterpret_cast<uint4*>(lrow + c0 + g * 8) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
                            }
                        }
                    }
                }
                if (i < a.Nq) a.lse[((int64_t)pr.b * a.H + pr.h) * a.Nq + i] = kLn2 * ((m - kPShift) + log2f(l));
                // the O_t reads above are complete (wait::ld); the next pair's first PV_t MMA waits for
                // this warpgroup's next P_t, so it cannot overwrite O_t earlier
            }
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == 8) tmem_dealloc(tmem, 512);
    if (threadIdx.x == 0 && *abort_flag) report_status(a.status, 1);
}

template <int D, bool BF16>
int launch(const fa_b200_params& p) {
    using Cfg = FwdCfg<D>;
    const CUtensorMapDataType dt = BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    CUtensorMap mq, mk, mv;
    int r;
    if ((r = cached_tmap_bnhd(&mq, p.q.ptr, dt, 2, p.B, p.Nq, p.H, D, p.q.stride_b, p.q.stride_n, p.q.stride_h, 128, 64, true)) ||
        (r = cached_tmap_bnhd(&mk, p.k.ptr, dt, 2, p.B, p.Nk, p.Hkv, D, p.k.stride_b, p.k.stride_n, p.k.stride_h, 128, 64, true)) ||
        (r = cached_tmap_bnhd(&mv, p.v.ptr, dt, 2, p.B, p.Nk, p.Hkv, D, p.v.stride_b, p.v.stride_n, p.v.stride_h, 128, 64, true))) {
        set_error("cuTensorMapEncodeTiled failed (%d)", r);
        return FA_ECUDA;
    }
    FwdArgs a;
    a.o = p.o.ptr;
    a.o_sb = p.o.stride_b; a.o_sn = p.o.stride_n; a.o_sh = p.o.stride_h;
    a.o_lo = p.o_lo.ptr;
    a.l_sb = p.o_lo.stride_b; a.l_sn = p.o_lo.stride_n; a.l_sh = p.o_lo.stride_h;
    a.lse = p.lse;
    a.status = p.status_word;
    a.wait_limit_ms = p.wait_limit_ms;
    a.B = p.B; a.Nq = p.Nq; a.Nk = p.Nk; a.H = p.H; a.Hkv = p.Hkv;
    a.kv_len = p.kv_lengths;
    a.causal = p.causal;
    a.shift = p.causal ? p.causal_shift : 0;
    a.n_pairs = (p.Nq + 2 * kBlockM - 1) / (2 * kBlockM);
    a.items_per_head = p.causal ? (a.n_pairs + 1) / 2 : a.n_pairs;
    const int64_t n_items = (int64_t)a.items_per_head * p.B * p.H;
    if (n_items > 0x7fffffff) { set_error("too many work items"); return FA_EUNSUPPORTED; }
    a.n_items = (int)n_items;
    a.scale_log2 = p.scale * kLog2e;
    a.drop_thr = dropout_threshold(p.dropout_p);
    a.inv_keep = 1.f / (1.f - dropout_effective_p(p.dropout_p));
    a.key = philox_make_key(p.seed, p.offset);
    a.rng = dropout_origin_of(p);
    // dropout: with a bit buffer the call's keep bits are written there first (unless an earlier call
    // left them) and the kernel loads them
    int drop = a.drop_thr ? 1 : 0;
    a.mq = nullptr;
    a.nq_pad = (int)align_up((size_t)p.Nq, 128);
    a.n_kblocks = (int)(align_up((size_t)p.Nk, 128) / 128);
    const size_t bits_one = dropout_bits_bytes(p);
    if (drop && p.dropout_bits && p.dropout_bits_bytes >= bits_one) {
        if (!p.dropout_bits_ready) {
            void* by_key = p.dropout_bits_bytes >= 2 * bits_one ? (char*)p.dropout_bits + bits_one : nullptr;
            int rc = launch_dropout_bits(p, p.dropout_bits, by_key);
            if (rc) return rc;
        }
        a.mq = (const uint4*)p.dropout_bits;
        drop = 2;
    }
    auto kernel = drop == 2 ? fwd_sm100_kernel<D, BF16, 2> : (drop == 1 ? fwd_sm100_kernel<D, BF16, 1> : fwd_sm100_kernel<D, BF16, 0>);
    {
        static std::mutex mu;
        static uint64_t done[3] = {0, 0, 0};
        FA_CUDA_CHECK(set_smem_limit_once(kernel, Cfg::kSmemBytes, p.device, &done[drop], &mu));
    }
    const int sms = sm_count(p.device);
    if (sms <= 0) { set_error("cannot read the SM count of device %d", p.device); return FA_ECUDA; }
    const int grid = a.n_items < sms ? a.n_items : sms;     // one persistent CTA per SM
    kernel<<<grid, kThreads, Cfg::kSmemBytes, (cudaStream_t)p.stream>>>(mq, mk, mv, a);
    FA_CUDA_CHECK(cudaGetLastError());
    return FA_OK;
}

bool tensor_ok(const fa_b200_tensor& t, int64_t B, int64_t N, int64_t H) {
    if (((uintptr_t)t.ptr & 15u) != 0) return false;
    if (H > 1 && (t.stride_h % 8) != 0) return false;
    if (N > 1 && (t.stride_n % 8) != 0) return false;
    if (B > 1 && (t.stride_b % 8) != 0) return false;
    return true;
}

}  // namespace

// Which calls the tensor-core family covers.  `why` names the first reason it does not.
bool sm100_supports(const fa_b200_params& p, bool backward, const char** why) {
    if (p.dtype == FA_B200_F32) {
        // fp32: the forward has a tensor-core kernel (TF32 products taken three times); the backward is CUDA-core tiles
        if (backward) { *why = "the fp32 backward is served by the CUDA-core kernels"; return false; }
        return sm100_tf32_fwd_supports(p, why);
    }
    if (p.dtype != FA_B200_F16 && p.dtype != FA_B200_BF16) { *why = "dtype must be fp16, bf16 or fp32"; return false; }
    if (p.bias.ptr) { *why = "an additive bias is served by the CUDA-core kernels"; return false; }
    if (p.D != 64 && p.D != 128) { *why = "head_dim must be 64 or 128"; return false; }
    if (!(p.scale > 0.f) || !(p.scale < 1e30f)) { *why = "scale must be positive and finite"; return false; }
    if (p.B > 65535 || p.H > 65535) { *why = "batch and heads must be below 65536"; return false; }
    if (!tensor_ok(p.q, p.B, p.Nq, p.H) || !tensor_ok(p.k, p.B, p.Nk, p.Hkv) ||
        !tensor_ok(p.v, p.B, p.Nk, p.Hkv) || !tensor_ok(p.o, p.B, p.Nq, p.H) ||
        (p.o_lo.ptr && !tensor_ok(p.o_lo, p.B, p.Nq, p.H)) ||
        (backward && (!tensor_ok(p.d_o, p.B, p.Nq, p.H) || !tensor_ok(p.dq, p.B, p.Nq, p.H) ||
                      !tensor_ok(p.dk, p.B, p.Nk, p.Hkv) || !tensor_ok(p.dv, p.B, p.Nk, p.Hkv)))) {
        *why = "tensors must be 16-byte aligned with strides that are multiples of 8 elements";
        return false;
    }
    *why = "";
    return true;
}

int sm100_fwd(const fa_b200_params& p) {
    if (p.dtype == FA_B200_F32) return sm100_tf32_fwd(p);
    if (p.dtype == FA_B200_BF16) return p.D == 128 ? launch<128, true>(p) : launch<64, true>(p);
    return p.D == 128 ? launch<128, false>(p) : launch<64, false>(p);
}

}  // namespace fa
