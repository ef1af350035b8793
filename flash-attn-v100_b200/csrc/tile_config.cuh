// The one place the tensor-core kernels' tuned numbers live.  The kernels are compiled from these
// constants and fa_b200_tile_config() reports the same constants, so the table cannot disagree with
// the code.  Replaces the reference's run-time tuner and its per-bucket table
// (kernels/autotuning.py:289-474, config.py:288-348).  Every value is the best of an A/B on B200;
// the runs behind them are listed in the design notes.
#pragma once

namespace fa {
namespace tile {

constexpr int kBlockM = 128;            // query rows per tile
constexpr int kBlockN = 128;            // key rows per block

// ---- forward (fwd_sm100.cu) ---------------------------------------------------------------------
constexpr int kFwdQTilesPerCta = 2;     // two query tiles in flight: the softmax of one hides the MMAs of the other
constexpr int kFwdWarps = 12;           // 8 softmax + MMA + TMA + 2 converting (bf16) / spare (fp16) warps
constexpr int fwd_kv_stages(int D) { return D == 128 ? 2 : 4; }      // K and V rings: what 227 KB hold
constexpr int kFwdRegsSoftmax = 208;    // setmaxnreg split; best of 224/56, 216/72, 208/88, 200/104
constexpr int kFwdRegsOther = 88;
constexpr int kFwdPolyPeriod = 2;       // of every kFwdPolyPeriod groups of four exponentials, kFwdPolyCount
constexpr int kFwdPolyCount = 1;        //   evaluate two on the FMA pipes: 0 % 0.559 ms, 25 % 0.544, 50 % 0.563
constexpr int kFwdHalfSignalAt = 16;    // first half of P handed over after this many of the second half's exps
constexpr float kFwdRescaleLog2 = 8.f;  // the running maximum is refreshed when it grows by more than 2^8

// ---- backward (bwd_sm100.cu) --------------------------------------------------------------------
constexpr int kBwdWarpgroups = 4;       // elementwise warpgroups (2 -> 4: backward +11 %)
constexpr int kBwdWarps = 4 * kBwdWarpgroups + 4;                    // + MMA, TMA, 2 converting / spare warps
// ring depth of the streamed tiles: U is read by the first and the last MMA of its step (three
// stages took 16 % off the dQ kernel), W within one step; the key-stationary dropout instance at
// D = 128 gives 4 KB to its masks and keeps two and two
constexpr int bwd_u_stages(int D, bool masks) { return D == 64 ? 4 : (masks ? 2 : 3); }
constexpr int bwd_w_stages(int D) { return D == 64 ? 3 : 2; }
// the dQ kernel is launched programmatically behind the dK/dV kernel while one head's K and V take at
// most this many bytes (N = 4096 at D = 128: -1 % of the backward; longer sequences showed no gain)
constexpr long long kBwdOverlapMaxKvBytes = 4ll << 20;
// CTA order: (batch, head) columns per group such that a group's Q, K, V and dO fit this budget (half of L2)
constexpr long long kBwdGroupBytes = 64ll << 20;
// D = 64: one kernel for dK, dV and dQ (dQ tiles summed in global memory) unless the two-pass variant is asked for
constexpr bool bwd_one_kernel(int D) { return D == 64; }

}  // namespace tile
}  // namespace fa
