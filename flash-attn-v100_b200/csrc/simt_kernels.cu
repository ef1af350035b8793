// CUDA-core attention tiles: the shape-generic kernel family of the library.
//
// Serves what the tensor-core family does not: fp32 inputs (computed in exact
// fp32 FMA arithmetic, no TF32 rounding), head dims other than 64/128 (any
// D <= 128), grouped K/V heads.  Same math as the tensor-core family:
//
//   forward  (replaces kernels/forward_kernel.py:18-243 of the reference)
//     per 64-row query tile, for each 64-row key tile at or below the diagonal:
//       S = scale*Q.K^T, mask, m' = max(m, rowmax S), P = exp(S - m'),
//       l = exp(m - m')*l + rowsum P,  O = exp(m - m')*O + (P o Z).V
//     then O /= l and lse = m + log l.   Z is the dropout keep/scale mask.
//   backward (replaces kernels/backward_kernel.py:17-205)
//     delta = rowsum(dO o O);  P = exp(S - lse);  dP = dO.V^T;
//     dS = P o (dP o Z - delta);  dV = (P o Z)^T.dO;  dK = scale*dS^T.Q;
//     dQ = scale*dS.K
//   dK/dV come from a key-stationary pass and dQ from a query-stationary pass,
//   so every output element is owned by exactly one thread and accumulated in
//   a fixed order: results are bit-reproducible.
#include "fa_common.cuh"
#include <math.h>

namespace fa {
namespace {

constexpr int BM = 64;       // query rows per tile
constexpr int BN = 64;       // key rows per tile
constexpr int NT = 256;      // threads per block: 16 x 16, 4x4 micro-tiles
constexpr int SLD = BN + 1;  // padded row pitch of the score tiles
constexpr int MAXC = 8;      // output columns per thread: D <= 16*MAXC = 128

struct SimtArgs {
    fa_b200_tensor q, k, v, o, d_o, dq, dk, dv;
    fa_b200_tensor o_lo;   // optional residual of o (forward: written; backward: added to o for delta)
    fa_b200_tensor bias;   // fp32 (B, H, Nq, Nk) with broadcast strides; ptr = nullptr: none
    float* d_scores;       // optional dense (B, H, Nq, Nk) gradient of the scores
    const int32_t* kv_len; // optional per-batch key counts
    float* lse;
    float* delta;
    int B, Nq, Nk, H, Hkv, D;
    int causal;
    int shift;          // key j is visible to query i iff j <= i + shift
    float scale;
    uint32_t drop_thr;   // 0 = no dropout
    float inv_keep;      // 1 / (1 - effective p)
    PhiloxKey key;
    DropoutOrigin rng;
};

template <typename T>
__device__ __forceinline__ void load_tile(float* dst, int ld, const T* base, int64_t stride_n,
                                          int row0, int nrows, int D, int rows_in_tile) {
    for (int idx = threadIdx.x; idx < rows_in_tile * D; idx += NT) {
        int r = idx / D, c = idx - r * D;
        int gr = row0 + r;
        dst[r * ld + c] = (gr < nrows) ? to_f32<T>(base[(int64_t)gr * stride_n + c]) : 0.f;
    }
}

template <typename T>
__global__ void __launch_bounds__(NT) simt_fwd_kernel(SimtArgs a) {
    extern __shared__ float smem[];
    const int D = a.D, ld = D + 1;
    float* Qs = smem;
    float* Ks = Qs + BM * ld;
    float* Vs = Ks + BN * ld;
    float* Ss = Vs + BN * ld;
    float* row_m = Ss + BM * SLD;
    float* row_l = row_m + BM;
    float* row_a = row_l + BM;

    const int mt = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    const int hk = h / (a.H / a.Hkv);
    const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
    const int m0 = mt * BM;
    const uint32_t bh = dropout_column(a.rng, b, h);
    const float* bias_b = a.bias.ptr ? (const float*)a.bias.ptr + (int64_t)b * a.bias.stride_b + (int64_t)h * a.bias.stride_h
                                     : nullptr;

    const T* qb = (const T*)a.q.ptr + (int64_t)b * a.q.stride_b + (int64_t)h * a.q.stride_h;
    const T* kb = (const T*)a.k.ptr + (int64_t)b * a.k.stride_b + (int64_t)hk * a.k.stride_h;
    const T* vb = (const T*)a.v.ptr + (int64_t)b * a.v.stride_b + (int64_t)hk * a.v.stride_h;
    T* ob = (T*)a.o.ptr + (int64_t)b * a.o.stride_b + (int64_t)h * a.o.stride_h;

    load_tile<T>(Qs, ld, qb, a.q.stride_n, m0, a.Nq, D, BM);
    if (tid < BM) { row_m[tid] = -INFINITY; row_l[tid] = 0.f; }

    float oacc[4][MAXC];
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int c = 0; c < MAXC; ++c) oacc[r][c] = 0.f;

    const int nk = kv_len_of(a.kv_len, b, a.Nk);      // keys this batch entry attends to
    int kv_end = nk;
    if (a.causal && m0 + BM + a.shift < kv_end) kv_end = m0 + BM + a.shift;

    for (int n0 = 0; n0 < kv_end; n0 += BN) {
        __syncthreads();
        load_tile<T>(Ks, ld, kb, a.k.stride_n, n0, a.Nk, D, BN);
        load_tile<T>(Vs, ld, vb, a.v.stride_n, n0, a.Nk, D, BN);
        __syncthreads();

        float acc[4][4];
#pragma unroll
        for (int r = 0; r < 4; ++r)
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[r][c] = 0.f;
        for (int d = 0; d < D; ++d) {
            float qa[4], kk[4];
#pragma unroll
            for (int r = 0; r < 4; ++r) qa[r] = Qs[(ty * 4 + r) * ld + d];
#pragma unroll
            for (int c = 0; c < 4; ++c) kk[c] = Ks[(tx + 16 * c) * ld + d];
#pragma unroll
            for (int r = 0; r < 4; ++r)
#pragma unroll
                for (int c = 0; c < 4; ++c) acc[r][c] = fmaf(qa[r], kk[c], acc[r][c]);
        }
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            int i = m0 + ty * 4 + r;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                int j = n0 + tx + 16 * c;
                float s = acc[r][c] * a.scale;
                if (bias_b && i < a.Nq && j < nk) s += bias_b[(int64_t)i * a.bias.stride_n + j];
                if (j >= nk || (a.causal && j > i + a.shift)) s = -INFINITY;
                Ss[(ty * 4 + r) * SLD + tx + 16 * c] = s;
            }
        }
        __syncthreads();

        {   // online softmax: 4 threads per row, 16 consecutive keys each (one Philox block)
            const int row = tid >> 2, part = tid & 3;
            float* srow = Ss + row * SLD + part * 16;
            float mx = -INFINITY;
#pragma unroll
            for (int c = 0; c < 16; ++c) mx = fmaxf(mx, srow[c]);
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            const float m_old = row_m[row], l_old = row_l[row];
            const float m_new = fmaxf(m_old, mx);
            const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
            uint32_t keep = 0xFFFFu;
            if (a.drop_thr)
                keep = dropout_keep_bits(a.key, bh, (uint32_t)(m0 + row),
                                         (uint32_t)((n0 >> 4) + part), a.drop_thr);
            float sum = 0.f;
#pragma unroll
            for (int c = 0; c < 16; ++c) {
                float p = expf(srow[c] - m_use);
                sum += p;
                srow[c] = ((keep >> c) & 1u) ? p * a.inv_keep : 0.f;
            }
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);
            sum += __shfl_xor_sync(0xffffffffu, sum, 2);
            const float alpha = expf(m_old - m_use);
            __syncwarp();
            if (part == 0) {
                row_m[row] = m_new;
                row_l[row] = alpha * l_old + sum;
                row_a[row] = alpha;
            }
        }
        __syncthreads();

#pragma unroll
        for (int r = 0; r < 4; ++r) {
            float al = row_a[ty * 4 + r];
#pragma unroll
            for (int c = 0; c < MAXC; ++c) oacc[r][c] *= al;
        }
        for (int j = 0; j < BN; ++j) {
            float pr[4];
#pragma unroll
            for (int r = 0; r < 4; ++r) pr[r] = Ss[(ty * 4 + r) * SLD + j];
#pragma unroll
            for (int c = 0; c < MAXC; ++c) {
                int col = tx + 16 * c;
                if (col < D) {
                    float vv = Vs[j * ld + col];
#pragma unroll
                    for (int r = 0; r < 4; ++r) oacc[r][c] = fmaf(pr[r], vv, oacc[r][c]);
                }
            }
        }
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        int row = ty * 4 + r, i = m0 + row;
        if (i < a.Nq) {
            float inv = 1.f / row_l[row];
#pragma unroll
            for (int c = 0; c < MAXC; ++c) {
                int col = tx + 16 * c;
                if (col < D) {
                    const float x = oacc[r][c] * inv;
                    const T hi = from_f32<T>(x);
                    ob[(int64_t)i * a.o.stride_n + col] = hi;
                    if (a.o_lo.ptr)
                        ((T*)a.o_lo.ptr)[(int64_t)b * a.o_lo.stride_b + (int64_t)i * a.o_lo.stride_n +
                                         (int64_t)h * a.o_lo.stride_h + col] = from_f32<T>(x - to_f32<T>(hi));
                }
            }
        }
    }
    if (tid < BM && m0 + tid < a.Nq)
        a.lse[((int64_t)b * a.H + h) * a.Nq + m0 + tid] = row_m[tid] + logf(row_l[tid]);
}

// delta[b,h,i] = sum_d dO[b,i,h,d] * O[b,i,h,d]; one warp per row.
template <typename T>
__global__ void __launch_bounds__(256) simt_delta_kernel(SimtArgs a) {
    int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    int lane = threadIdx.x & 31;
    int64_t total = (int64_t)a.B * a.H * a.Nq;
    if (row >= total) return;
    int i = (int)(row % a.Nq);
    int h = (int)((row / a.Nq) % a.H);
    int b = (int)(row / ((int64_t)a.Nq * a.H));
    const T* o = (const T*)a.o.ptr + (int64_t)b * a.o.stride_b + (int64_t)i * a.o.stride_n + (int64_t)h * a.o.stride_h;
    const T* g = (const T*)a.d_o.ptr + (int64_t)b * a.d_o.stride_b + (int64_t)i * a.d_o.stride_n + (int64_t)h * a.d_o.stride_h;
    float s = 0.f;
    if (a.o_lo.ptr) {
        const T* l = (const T*)a.o_lo.ptr + (int64_t)b * a.o_lo.stride_b + (int64_t)i * a.o_lo.stride_n + (int64_t)h * a.o_lo.stride_h;
        for (int d = lane; d < a.D; d += 32) s = fmaf(to_f32<T>(o[d]) + to_f32<T>(l[d]), to_f32<T>(g[d]), s);
    } else {
        for (int d = lane; d < a.D; d += 32) s = fmaf(to_f32<T>(o[d]), to_f32<T>(g[d]), s);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
    if (lane == 0) a.delta[row] = s;
}

// MODE 0: key-stationary, writes dK and dV.  MODE 1: query-stationary, writes dQ.
template <typename T, int MODE>
__global__ void __launch_bounds__(NT) simt_bwd_kernel(SimtArgs a) {
    extern __shared__ float smem[];
    const int D = a.D, ld = D + 1;
    float* Qs = smem;
    float* Gs = Qs + BM * ld;    // dO tile
    float* Ks = Gs + BM * ld;
    float* Vs = Ks + BN * ld;
    float* Ps = Vs + BN * ld;    // P o Z
    float* Ds = Ps + BM * SLD;   // dS
    float* lse_s = Ds + BM * SLD;
    float* del_s = lse_s + BM;

    const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
    const int b = blockIdx.z;
    const int group = a.H / a.Hkv;

    float acc0[4][MAXC], acc1[4][MAXC];   // MODE 0: dK, dV.  MODE 1: dQ, unused.
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int c = 0; c < MAXC; ++c) { acc0[r][c] = 0.f; acc1[r][c] = 0.f; }

    const int tile = blockIdx.x;
    const int nk = kv_len_of(a.kv_len, b, a.Nk);      // keys this batch entry attends to
    const int hk = (MODE == 0) ? blockIdx.y : blockIdx.y / group;
    const int h_begin = (MODE == 0) ? hk * group : blockIdx.y;
    const int h_end = (MODE == 0) ? h_begin + group : h_begin + 1;

    const T* kb = (const T*)a.k.ptr + (int64_t)b * a.k.stride_b + (int64_t)hk * a.k.stride_h;
    const T* vb = (const T*)a.v.ptr + (int64_t)b * a.v.stride_b + (int64_t)hk * a.v.stride_h;

    if (MODE == 0) {
        load_tile<T>(Ks, ld, kb, a.k.stride_n, tile * BN, a.Nk, D, BN);
        load_tile<T>(Vs, ld, vb, a.v.stride_n, tile * BN, a.Nk, D, BN);
    }

    for (int h = h_begin; h < h_end; ++h) {
        const uint32_t bh = dropout_column(a.rng, b, h);
        const T* qb = (const T*)a.q.ptr + (int64_t)b * a.q.stride_b + (int64_t)h * a.q.stride_h;
        const T* gb = (const T*)a.d_o.ptr + (int64_t)b * a.d_o.stride_b + (int64_t)h * a.d_o.stride_h;
        const float* lse_b = a.lse + ((int64_t)b * a.H + h) * a.Nq;
        const float* del_b = a.delta + ((int64_t)b * a.H + h) * a.Nq;
        const float* bias_b = a.bias.ptr ? (const float*)a.bias.ptr + (int64_t)b * a.bias.stride_b +
                                               (int64_t)h * a.bias.stride_h : nullptr;
        float* ds_b = a.d_scores ? a.d_scores + ((int64_t)b * a.H + h) * (int64_t)a.Nq * a.Nk : nullptr;

        int it_begin, it_end;   // tile indices of the streamed operand
        if (MODE == 0) {
            it_begin = (a.causal && tile * BN > a.shift) ? (tile * BN - a.shift) / BM : 0;
            it_end = (a.Nq + BM - 1) / BM;
        } else {
            int kv_end = nk;
            if (a.causal && tile * BM + BM + a.shift < kv_end) kv_end = tile * BM + BM + a.shift;
            it_begin = 0;
            it_end = (kv_end + BN - 1) / BN;
        }
        if (MODE == 1) {
            __syncthreads();
            load_tile<T>(Qs, ld, qb, a.q.stride_n, tile * BM, a.Nq, D, BM);
            load_tile<T>(Gs, ld, gb, a.d_o.stride_n, tile * BM, a.Nq, D, BM);
            if (tid < BM) {
                int i = tile * BM + tid;
                lse_s[tid] = (i < a.Nq) ? lse_b[i] : 0.f;
                del_s[tid] = (i < a.Nq) ? del_b[i] : 0.f;
            }
        }

        for (int it = it_begin; it < it_end; ++it) {
            const int m0 = (MODE == 0) ? it * BM : tile * BM;
            const int n0 = (MODE == 0) ? tile * BN : it * BN;
            __syncthreads();
            if (MODE == 0) {
                load_tile<T>(Qs, ld, qb, a.q.stride_n, m0, a.Nq, D, BM);
                load_tile<T>(Gs, ld, gb, a.d_o.stride_n, m0, a.Nq, D, BM);
                if (tid < BM) {
                    int i = m0 + tid;
                    lse_s[tid] = (i < a.Nq) ? lse_b[i] : 0.f;
                    del_s[tid] = (i < a.Nq) ? del_b[i] : 0.f;
                }
            } else {
                load_tile<T>(Ks, ld, kb, a.k.stride_n, n0, a.Nk, D, BN);
                load_tile<T>(Vs, ld, vb, a.v.stride_n, n0, a.Nk, D, BN);
            }
            __syncthreads();

            float s_acc[4][4], p_acc[4][4];
#pragma unroll
            for (int r = 0; r < 4; ++r)
#pragma unroll
                for (int c = 0; c < 4; ++c) { s_acc[r][c] = 0.f; p_acc[r][c] = 0.f; }
            for (int d = 0; d < D; ++d) {
                float qa[4], ga[4], kk[4], vv[4];
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    qa[r] = Qs[(ty * 4 + r) * ld + d];
                    ga[r] = Gs[(ty * 4 + r) * ld + d];
                }
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    kk[c] = Ks[(tx + 16 * c) * ld + d];
                    vv[c] = Vs[(tx + 16 * c) * ld + d];
                }
#pragma unroll
                for (int r = 0; r < 4; ++r)
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        s_acc[r][c] = fmaf(qa[r], kk[c], s_acc[r][c]);
                        p_acc[r][c] = fmaf(ga[r], vv[c], p_acc[r][c]);
                    }
            }
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const int row = ty * 4 + r, i = m0 + row;
                const float lse_i = lse_s[row], del_i = del_s[row];
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const int col = tx + 16 * c, j = n0 + col;
                    float p = 0.f, z = 1.f;
                    bool visible = (i < a.Nq) && (j < nk) && !(a.causal && j > i + a.shift);
                    if (visible) {
                        float s = s_acc[r][c] * a.scale;
                        if (bias_b) s += bias_b[(int64_t)i * a.bias.stride_n + j];
                        p = expf(s - lse_i);
                    }
                    if (a.drop_thr)
                        z = dropout_keep(a.key, bh, (uint32_t)i, (uint32_t)j, a.drop_thr) ? a.inv_keep : 0.f;
                    Ps[row * SLD + col] = p * z;
                    const float ds = p * (p_acc[r][c] * z - del_i);
                    Ds[row * SLD + col] = ds;
                    if (MODE == 1 && ds_b && visible) ds_b[(int64_t)i * a.Nk + j] = ds;
                }
            }
            __syncthreads();

            if (MODE == 0) {
                // rows of the accumulators are keys j = ty*4+r of this tile
                for (int i = 0; i < BM; ++i) {
                    float pz[4], ds[4];
#pragma unroll
                    for (int r = 0; r < 4; ++r) {
                        pz[r] = Ps[i * SLD + ty * 4 + r];
                        ds[r] = Ds[i * SLD + ty * 4 + r];
                    }
#pragma unroll
                    for (int c = 0; c < MAXC; ++c) {
                        int col = tx + 16 * c;
                        if (col < D) {
                            float g = Gs[i * ld + col], q = Qs[i * ld + col];
#pragma unroll
                            for (int r = 0; r < 4; ++r) {
                                acc1[r][c] = fmaf(pz[r], g, acc1[r][c]);
                                acc0[r][c] = fmaf(ds[r], q, acc0[r][c]);
                            }
                        }
                    }
                }
            } else {
                for (int j = 0; j < BN; ++j) {
                    float ds[4];
#pragma unroll
                    for (int r = 0; r < 4; ++r) ds[r] = Ds[(ty * 4 + r) * SLD + j];
#pragma unroll
                    for (int c = 0; c < MAXC; ++c) {
                        int col = tx + 16 * c;
                        if (col < D) {
                            float kk = Ks[j * ld + col];
#pragma unroll
                            for (int r = 0; r < 4; ++r) acc0[r][c] = fmaf(ds[r], kk, acc0[r][c]);
                        }
                    }
                }
            }
        }
    }

    if (MODE == 0) {
        T* dkb = (T*)a.dk.ptr + (int64_t)b * a.dk.stride_b + (int64_t)hk * a.dk.stride_h;
        T* dvb = (T*)a.dv.ptr + (int64_t)b * a.dv.stride_b + (int64_t)hk * a.dv.stride_h;
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            int j = tile * BN + ty * 4 + r;
            if (j < a.Nk) {
#pragma unroll
                for (int c = 0; c < MAXC; ++c) {
                    int col = tx + 16 * c;
                    if (col < D) {
                        dkb[(int64_t)j * a.dk.stride_n + col] = from_f32<T>(acc0[r][c] * a.scale);
                        dvb[(int64_t)j * a.dv.stride_n + col] = from_f32<T>(acc1[r][c]);
                    }
                }
            }
        }
    } else {
        const int h = blockIdx.y;
        T* dqb = (T*)a.dq.ptr + (int64_t)b * a.dq.stride_b + (int64_t)h * a.dq.stride_h;
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            int i = tile * BM + ty * 4 + r;
            if (i < a.Nq) {
#pragma unroll
                for (int c = 0; c < MAXC; ++c) {
                    int col = tx + 16 * c;
                    if (col < D) dqb[(int64_t)i * a.dq.stride_n + col] = from_f32<T>(acc0[r][c] * a.scale);
                }
            }
        }
    }
}

__global__ void dropout_mask_kernel(PhiloxKey key, uint32_t thr, int H, int Nq, int Nk,
                                    int64_t n_blocks16, uint8_t* out) {
    // one thread per (b*H+h, i, 16-key block)
    int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= n_blocks16) return;
    int jb_per_row = (Nk + 15) / 16;
    int jb = (int)(t % jb_per_row);
    int64_t rowid = t / jb_per_row;
    int i = (int)(rowid % Nq);
    uint32_t bh = (uint32_t)(rowid / Nq);
    uint32_t bits = thr ? dropout_keep_bits(key, bh, (uint32_t)i, (uint32_t)jb, thr) : 0xFFFFu;
    uint8_t* dst = out + rowid * Nk + (int64_t)jb * 16;
    for (int c = 0; c < 16 && jb * 16 + c < Nk; ++c) dst[c] = (bits >> c) & 1u;
}

// Transpose of a 32 x 32 bit matrix held one row per lane: afterwards lane k holds column k, bit q = the
// bit lane q held at position k.  Five exchanges of half-blocks (16, 8, 4, 2, 1 wide).
__device__ __forceinline__ uint32_t transpose_bits_32x32(uint32_t x, int lane) {
    const uint32_t masks[5] = {0x0000FFFFu, 0x00FF00FFu, 0x0F0F0F0Fu, 0x33333333u, 0x55555555u};
#pragma unroll
    for (int t = 0; t < 5; ++t) {
        const int s = 16 >> t;
        const uint32_t m = masks[t];
        const uint32_t y = __shfl_xor_sync(0xffffffffu, x, s);
        x = (lane & s) ? ((x & ~m) | ((y & ~m) >> s)) : ((x & m) | ((y & m) << s));
    }
    return x;
}

// The keep bits of a whole call, written once for the tensor-core kernels to load (drawing them inside
// those kernels costs their softmax / elementwise threads as many instructions as the attention math
// itself; here every SM draws at full integer rate, and the forward's bits serve the backward too).
// One warp per (column, 32 queries, 128 keys): lane = query, eight Philox blocks of 16 keys each.
//   mq[(col * NJ + j128) * nq_pad + i]            uint4: bit c of the 128 = key j128*128 + c   (query-major)
//   mk[((col * NI + i128) * 4 + g) * nk_pad + k]  uint32: bit q = query i128*128 + 32 g + q     (key-major:
//       the 32 x 32 transposes of the warp's four words)
// Tiles the causal mask hides completely hold no bits (nobody reads them: P is zero there).  Under the
// usual mask (square, key j visible to query i iff j <= i) the 32-query blocks are dealt in pairs, block p
// with block NIB-1-p: together they have NJ + 1 live key blocks whatever p, so every warp of the grid has
// work (a grid over all (block, key block) items, half of them hidden, measured 0.36 against 0.33 ms on
// B32 H16 N2048; a fixed grid that strides over the items 0.56 ms).  Other shapes walk all items and skip.
__global__ void __launch_bounds__(256, 8)
dropout_bits_kernel(PhiloxKey key, uint32_t thr, DropoutOrigin rng, int H, int Nq, int nq_pad, int nk_pad,
                    int causal, int shift, int paired, int64_t n_items, uint4* __restrict__ mq,
                    uint32_t* __restrict__ mk) {
    const int lane = threadIdx.x & 31;
    const int64_t item = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (item >= n_items) return;                                     // whole warps leave together
    const int NJ = nk_pad / 128, NIB = nq_pad / 32;
    int j128, ib;
    int64_t col;                                                      // local b * H + h
    if (paired) {
        const int s = (int)(item % (NJ + 1));
        const int64_t rest = item / (NJ + 1);
        const int pr = (int)(rest % (NIB / 2));
        col = rest / (NIB / 2);
        const int live_lo = pr / 4 + 1;                               // live key blocks of the pair's first block
        ib = s < live_lo ? pr : NIB - 1 - pr;
        j128 = s < live_lo ? s : s - live_lo;
    } else {
        j128 = (int)(item % NJ);
        const int64_t rest = item / NJ;
        ib = (int)(rest % NIB);
        col = rest / NIB;
        if (causal && (int64_t)j128 * 128 > (int64_t)ib * 32 + 31 + shift) return;
    }
    const int i = ib * 32 + lane;
    const uint32_t column = dropout_column(rng, (int)(col / H), (int)(col % H));
    uint32_t w4[4] = {0u, 0u, 0u, 0u};
#pragma unroll
    for (int g = 0; g < 8; ++g)
        w4[g >> 1] |= dropout_keep_bits(key, column, (uint32_t)i, (uint32_t)(j128 * 8 + g), thr) << (16 * (g & 1));
    if (mq) mq[(col * NJ + j128) * (int64_t)nq_pad + i] = make_uint4(w4[0], w4[1], w4[2], w4[3]);
    if (mk) {
        uint32_t* dst = mk + ((col * (nq_pad / 128) + (ib >> 2)) * 4 + (ib & 3)) * (int64_t)nk_pad + j128 * 128 + lane;
#pragma unroll
        for (int x = 0; x < 4; ++x) dst[32 * x] = transpose_bits_32x32(w4[x], lane);
    }
}

SimtArgs make_args(const fa_b200_params& p, float* delta) {
    SimtArgs a;
    a.q = p.q; a.k = p.k; a.v = p.v; a.o = p.o; a.d_o = p.d_o; a.dq = p.dq; a.dk = p.dk; a.dv = p.dv;
    a.o_lo = p.o_lo;
    a.lse = p.lse; a.delta = delta;
    a.bias = p.bias; a.d_scores = p.d_scores; a.kv_len = p.kv_lengths;
    a.B = p.B; a.Nq = p.Nq; a.Nk = p.Nk; a.H = p.H; a.Hkv = p.Hkv; a.D = p.D;
    a.causal = p.causal; a.shift = p.causal ? p.causal_shift : 0; a.scale = p.scale;
    a.drop_thr = dropout_threshold(p.dropout_p);
    a.inv_keep = 1.f / (1.f - dropout_effective_p(p.dropout_p));
    a.key = philox_make_key(p.seed, p.offset);
    a.rng = dropout_origin_of(p);
    return a;
}

template <typename K>
int set_smem(K kernel, size_t bytes) {
    FA_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
    return FA_OK;
}

template <typename T>
int launch_fwd(const fa_b200_params& p) {
    SimtArgs a = make_args(p, nullptr);
    size_t smem = ((size_t)(BM + 2 * BN) * (p.D + 1) + (size_t)BM * SLD + 3 * BM) * sizeof(float);
    int rc = set_smem(simt_fwd_kernel<T>, smem);
    if (rc) return rc;
    dim3 grid((p.Nq + BM - 1) / BM, p.H, p.B);
    simt_fwd_kernel<T><<<grid, NT, smem, (cudaStream_t)p.stream>>>(a);
    FA_CUDA_CHECK(cudaGetLastError());
    return FA_OK;
}

template <typename T>
int launch_bwd(const fa_b200_params& p, const BwdWorkspace& ws) {
    float* delta = (float*)((char*)p.workspace + ws.delta_off);
    SimtArgs a = make_args(p, delta);
    cudaStream_t st = (cudaStream_t)p.stream;
    int64_t rows = (int64_t)p.B * p.H * p.Nq;
    const int phases = p.bwd_phases ? p.bwd_phases : 7;
    if (phases & 1) {
        simt_delta_kernel<T><<<(unsigned)((rows + 7) / 8), 256, 0, st>>>(a);
        FA_CUDA_CHECK(cudaGetLastError());
    }
    size_t smem = ((size_t)(2 * BM + 2 * BN) * (p.D + 1) + (size_t)2 * BM * SLD + 2 * BM) * sizeof(float);
    int rc = set_smem(simt_bwd_kernel<T, 0>, smem);
    if (rc) return rc;
    rc = set_smem(simt_bwd_kernel<T, 1>, smem);
    if (rc) return rc;
    if (phases & 2) {
        dim3 grid_kv((p.Nk + BN - 1) / BN, p.Hkv, p.B);
        simt_bwd_kernel<T, 0><<<grid_kv, NT, smem, st>>>(a);
        FA_CUDA_CHECK(cudaGetLastError());
    }
    if (phases & 4) {
        dim3 grid_q((p.Nq + BM - 1) / BM, p.H, p.B);
        simt_bwd_kernel<T, 1><<<grid_q, NT, smem, st>>>(a);
        FA_CUDA_CHECK(cudaGetLastError());
    }
    return FA_OK;
}

}  // namespace

bool simt_supports(const fa_b200_params& p) { return p.D >= 1 && p.D <= 16 * MAXC; }

int simt_fwd(const fa_b200_params& p) {
    switch (p.dtype) {
        case FA_B200_F16:  return launch_fwd<__half>(p);
        case FA_B200_BF16: return launch_fwd<__nv_bfloat16>(p);
        case FA_B200_F32:  return launch_fwd<float>(p);
    }
    return FA_EINVAL;
}

int simt_bwd(const fa_b200_params& p, const BwdWorkspace& ws) {
    switch (p.dtype) {
        case FA_B200_F16:  return launch_bwd<__half>(p, ws);
        case FA_B200_BF16: return launch_bwd<__nv_bfloat16>(p, ws);
        case FA_B200_F32:  return launch_bwd<float>(p, ws);
    }
    return FA_EINVAL;
}

// Bytes of one orientation of a call's keep bits: B*H columns x ceil128(Nq) x ceil128(Nk) bits.
size_t dropout_bits_bytes(const fa_b200_params& p) {
    return (size_t)p.B * p.H * align_up((size_t)p.Nq, 128) * (align_up((size_t)p.Nk, 128) / 8);
}

int launch_dropout_bits(const fa_b200_params& p, void* mq, void* mk) {
    const int nq_pad = (int)align_up((size_t)p.Nq, 128), nk_pad = (int)align_up((size_t)p.Nk, 128);
    const int shift = p.causal ? p.causal_shift : 0;
    // the usual causal mask on a square problem: pairs of query blocks, no hidden items (see the kernel)
    const int paired = (p.causal && shift == 0 && nq_pad == nk_pad) ? 1 : 0;
    const int64_t per_column = paired ? (int64_t)(nq_pad / 64) * (nk_pad / 128 + 1) : (int64_t)(nq_pad / 32) * (nk_pad / 128);
    const int64_t n_items = (int64_t)p.B * p.H * per_column;
    const int64_t blocks = (n_items + 7) / 8;
    if (blocks > 0x7fffffff) { set_error("problem too large for the dropout-bits grid"); return FA_EUNSUPPORTED; }
    if (blocks == 0 || (!mq && !mk)) return FA_OK;
    dropout_bits_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)p.stream>>>(
        philox_make_key(p.seed, p.offset), dropout_threshold(p.dropout_p), dropout_origin_of(p), p.H, p.Nq, nq_pad,
        nk_pad, p.causal, shift, paired, n_items, (uint4*)mq, (uint32_t*)mk);
    FA_CUDA_CHECK(cudaGetLastError());
    return FA_OK;
}

int launch_dropout_mask(uint64_t seed, uint64_t offset, float p, int B, int H, int Nq, int Nk,
                        uint8_t* out, cudaStream_t stream) {
    int64_t n = (int64_t)B * H * Nq * ((Nk + 15) / 16);
    if (n == 0) return FA_OK;
    dropout_mask_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(
        philox_make_key(seed, offset), dropout_threshold(p), H, Nq, Nk, n, out);
    FA_CUDA_CHECK(cudaGetLastError());
    return FA_OK;
}

}  // namespace fa
