/*
 * cpu_ref.c — plain-C restatement of the attention hot path, in double
 * precision.  TEST INFRASTRUCTURE: only tests/, __graft_entry__.smoke() and
 * bench.py's CPU-baseline leg may load the library built from this file; the
 * shipped package never does.
 *
 * Forward follows the reference's math path, __init__.py:36-54:
 *   scores = (q*scale).k^T  (:41)   causal: j > i -> -inf (:43-48); `causal` = 1 + shift hides
 *   j > i + shift instead (shift 0 is the reference's mask, Nk - Nq the bottom-right alignment)
 *   P = softmax(scores) (:50)       O = P.v (:51)
 * on (B, N, H, D) contiguous float inputs (:34-38 transposes are index math
 * here).  Dropout follows the reference's test twin,
 * tests/test_attention.py:69-73: P is dropped after normalisation and kept
 * entries are scaled by 1/(1-p); the keep mask is an input.  LSE and the
 * backward pass have no counterpart in the reference math path (its LSE is a
 * dummy, tests/test_attention.py:81-85); they restate the standard
 * identities
 *   lse_i = log sum_j exp(s_ij);  delta_i = sum_d dO_id O_id
 *   dV = (PoZ)^T dO;  dP = dO V^T;  dS = P o (dP o Z - delta)
 *   dQ = scale dS K;  dK = scale dS^T Q.
 *
 * The Philox4x32-10 block function is restated independently of the
 * library's (from Salmon et al., SC'11) so that the two can be compared.
 *
 * Build: see oracle/Makefile (gcc -O2 -shared -fPIC).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define IDX(b, n, h, d, N, H, D) ((((int64_t)(b) * (N) + (n)) * (H) + (h)) * (D) + (d))

/* scores row i of head (b,h) into s[0..Nk) (double), returns lse */
static double score_row(const float* q, const float* k, int b, int h, int hk, int i,
                        int Nq, int Nk, int H, int Hkv, int D, int causal, double scale, double* s) {
    double mx = -INFINITY;
    for (int j = 0; j < Nk; ++j) {
        if (causal && j > i + (causal - 1)) { s[j] = -INFINITY; continue; }
        double acc = 0.0;
        for (int d = 0; d < D; ++d)
            acc += ((double)q[IDX(b, i, h, d, Nq, H, D)] * scale) * (double)k[IDX(b, j, hk, d, Nk, Hkv, D)];
        s[j] = acc;
        if (acc > mx) mx = acc;
    }
    double sum = 0.0;
    for (int j = 0; j < Nk; ++j) sum += exp(s[j] - mx);
    return mx + log(sum);
}

/* keep: (B,H,Nq,Nk) bytes or NULL.  o: (B,Nq,H,D) float, lse: (B,H,Nq) float */
int fa_oracle_forward(const float* q, const float* k, const float* v,
                      int B, int Nq, int Nk, int H, int Hkv, int D,
                      int causal, double scale, const uint8_t* keep, double dropout_p,
                      float* o, float* lse) {
    if (H % Hkv) return -1;
    int g = H / Hkv;
    double zscale = 1.0 / (1.0 - dropout_p);
    for (int b = 0; b < B; ++b)
        for (int h = 0; h < H; ++h) {
            double* s = (double*)malloc(sizeof(double) * (size_t)(Nk + D));
            double* acc = s + Nk;
            int hk = h / g;
            for (int i = 0; i < Nq; ++i) {
                double l = score_row(q, k, b, h, hk, i, Nq, Nk, H, Hkv, D, causal, scale, s);
                lse[((int64_t)b * H + h) * Nq + i] = (float)l;
                for (int d = 0; d < D; ++d) acc[d] = 0.0;
                const uint8_t* kr = keep ? keep + (((int64_t)b * H + h) * Nq + i) * Nk : NULL;
                for (int j = 0; j < Nk; ++j) {
                    double p = exp(s[j] - l);
                    if (kr) p = kr[j] ? p * zscale : 0.0;
                    if (p == 0.0) continue;
                    for (int d = 0; d < D; ++d) acc[d] += p * (double)v[IDX(b, j, hk, d, Nk, Hkv, D)];
                }
                for (int d = 0; d < D; ++d) o[IDX(b, i, h, d, Nq, H, D)] = (float)acc[d];
            }
            free(s);
        }
    return 0;
}

/* dq (B,Nq,H,D), dk, dv (B,Nk,Hkv,D) float outputs; o and lse from forward */
int fa_oracle_backward(const float* q, const float* k, const float* v, const float* o,
                       const float* lse, const float* d_o,
                       int B, int Nq, int Nk, int H, int Hkv, int D,
                       int causal, double scale, const uint8_t* keep, double dropout_p,
                       float* dq, float* dk, float* dv) {
    if (H % Hkv) return -1;
    int g = H / Hkv;
    double zscale = 1.0 / (1.0 - dropout_p);
    for (int b = 0; b < B; ++b)
        for (int hk = 0; hk < Hkv; ++hk) {
            size_t nkd = (size_t)Nk * D;
            double* dka = (double*)calloc(2 * nkd + (size_t)Nk + D, sizeof(double));
            double* dva = dka + nkd;
            double* s = dva + nkd;
            double* dqa = s + Nk;
            for (int h = hk * g; h < (hk + 1) * g; ++h)
                for (int i = 0; i < Nq; ++i) {
                    score_row(q, k, b, h, hk, i, Nq, Nk, H, Hkv, D, causal, scale, s);
                    double l = (double)lse[((int64_t)b * H + h) * Nq + i];
                    double delta = 0.0;
                    for (int d = 0; d < D; ++d)
                        delta += (double)d_o[IDX(b, i, h, d, Nq, H, D)] * (double)o[IDX(b, i, h, d, Nq, H, D)];
                    for (int d = 0; d < D; ++d) dqa[d] = 0.0;
                    const uint8_t* kr = keep ? keep + (((int64_t)b * H + h) * Nq + i) * Nk : NULL;
                    for (int j = 0; j < Nk; ++j) {
                        if (causal && j > i + (causal - 1)) continue;
                        double p = exp(s[j] - l);
                        double z = kr ? (kr[j] ? zscale : 0.0) : 1.0;
                        double dp = 0.0;
                        for (int d = 0; d < D; ++d)
                            dp += (double)d_o[IDX(b, i, h, d, Nq, H, D)] * (double)v[IDX(b, j, hk, d, Nk, Hkv, D)];
                        double ds = p * (dp * z - delta);
                        for (int d = 0; d < D; ++d) {
                            dva[(size_t)j * D + d] += p * z * (double)d_o[IDX(b, i, h, d, Nq, H, D)];
                            dka[(size_t)j * D + d] += scale * ds * (double)q[IDX(b, i, h, d, Nq, H, D)];
                            dqa[d] += scale * ds * (double)k[IDX(b, j, hk, d, Nk, Hkv, D)];
                        }
                    }
                    for (int d = 0; d < D; ++d) dq[IDX(b, i, h, d, Nq, H, D)] = (float)dqa[d];
                }
            for (int j = 0; j < Nk; ++j)
                for (int d = 0; d < D; ++d) {
                    dk[IDX(b, j, hk, d, Nk, Hkv, D)] = (float)dka[(size_t)j * D + d];
                    dv[IDX(b, j, hk, d, Nk, Hkv, D)] = (float)dva[(size_t)j * D + d];
                }
            free(dka);
        }
    return 0;
}

/* Philox4x32-10, restated from the SC'11 paper (Figure / section 3.2). */
void fa_oracle_philox4x32_10(const uint32_t ctr[4], const uint32_t key[2], uint32_t out[4]) {
    uint32_t c0 = ctr[0], c1 = ctr[1], c2 = ctr[2], c3 = ctr[3];
    uint32_t k0 = key[0], k1 = key[1];
    for (int round = 0; round < 10; ++round) {
        if (round > 0) { k0 += 0x9E3779B9u; k1 += 0xBB67AE85u; }
        uint64_t p0 = (uint64_t)0xD2511F53u * c0;
        uint64_t p1 = (uint64_t)0xCD9E8D57u * c2;
        uint32_t n0 = (uint32_t)(p1 >> 32) ^ c1 ^ k0;
        uint32_t n1 = (uint32_t)p1;
        uint32_t n2 = (uint32_t)(p0 >> 32) ^ c3 ^ k1;
        uint32_t n3 = (uint32_t)p0;
        c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    }
    out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

/* Keep mask of the library's dropout stream, written from its stated
 * definition: block counter = (j/16, i, b*H+h, offset_lo), key = (seed_lo,
 * seed_hi ^ offset_hi), byte j%16 (little-endian over the 4 words) >=
 * round(p*256) keeps. */
void fa_oracle_dropout_mask(uint64_t seed, uint64_t offset, double p,
                            int B, int H, int Nq, int Nk, uint8_t* out) {
    uint32_t thr = 0;
    if (p > 0.0) { thr = (uint32_t)(p * 256.0 + 0.5); if (thr > 255) thr = 255; }
    uint32_t key[2] = { (uint32_t)seed, (uint32_t)(seed >> 32) ^ (uint32_t)(offset >> 32) };
    for (int64_t row = 0; row < (int64_t)B * H * Nq; ++row) {
        uint32_t bh = (uint32_t)(row / Nq), i = (uint32_t)(row % Nq);
        for (int j = 0; j < Nk; ++j) {
            uint32_t ctr[4] = { (uint32_t)(j / 16), i, bh, (uint32_t)offset }, w[4];
            fa_oracle_philox4x32_10(ctr, key, w);
            uint32_t t = (uint32_t)(j % 16);
            uint32_t byte = (w[t / 4] >> (8 * (t % 4))) & 0xFFu;
            out[row * Nk + j] = (thr == 0 || byte >= thr) ? 1 : 0;
        }
    }
}
