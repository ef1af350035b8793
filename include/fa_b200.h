/*
 * fa_b200.h — C ABI of libfa_b200.so: exact attention forward/backward for
 * NVIDIA B200 (sm_100a).
 *
 * The reference project (mini-kio/flash-attn-v100) is pure Python and has no
 * FFI of its own: its host code launches two Triton kernels directly
 *   kernels/forward_kernel.py:246-387   flash_attention_forward_triton_enhanced
 *   kernels/backward_kernel.py:208-318  flash_attention_backward_triton_enhanced
 * passing raw pointers, the six sizes and per-tensor (batch, head, seq, dim)
 * strides (kernels/forward_kernel.py:349-385).  The entry points below are the
 * C-ABI counterpart of those two launchers plus the small amount of state the
 * launchers derive on the host (tile choice, workspace size, dropout stream).
 *
 * Conventions
 *  - Tensors q, k, v, o, dO, dQ, dK, dV use the reference's (B, N, H, D)
 *    layout (interface.py:228-230).  The D axis must be contiguous; the batch,
 *    sequence and head strides are given in ELEMENTS, so head- or batch-sliced
 *    views are consumed in place.
 *  - lse is (B, H, Nq) float32, contiguous, natural-log log-sum-exp of the
 *    scaled, masked scores (the reference's return_softmax_lse output,
 *    ops/attention.py:229-230).
 *  - Every pointer is a device pointer on `device`, borrowed for the duration
 *    of the enqueued work.  The library allocates no device memory; scratch is
 *    passed in through `workspace`.
 *  - Work is enqueued on `stream` (a cudaStream_t); no call synchronises.
 *  - Functions return FA_OK or a negative fa_b200_status; they never throw or
 *    abort.  fa_b200_strerror() describes a code, fa_b200_last_error() the
 *    detail of the last failure on the calling thread.
 */
#ifndef FA_B200_H
#define FA_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FA_B200_ABI_VERSION 3

typedef enum fa_b200_dtype {
    FA_B200_F16  = 0,
    FA_B200_BF16 = 1,
    FA_B200_F32  = 2
} fa_b200_dtype;

typedef enum fa_b200_status {
    FA_OK           =  0,
    FA_EINVAL       = -1,  /* null pointer, bad size, bad enum, bad struct_bytes   */
    FA_EUNSUPPORTED = -2,  /* shape/dtype combination no kernel covers             */
    FA_EALIGN       = -3,  /* pointer or stride alignment the chosen kernel needs  */
    FA_EWORKSPACE   = -4,  /* workspace missing or too small                       */
    FA_ECUDA        = -5,  /* a CUDA runtime/driver call failed                    */
    FA_ETIMEOUT     = -6   /* a bounded device-side wait ran out (status word)     */
} fa_b200_status;

/* Which kernel family serves the call.  AUTO: the tensor-core family where it covers the call
 * (fp16/bf16, D in {64, 128}, aligned tensors, no bias), in its deterministic form, else CUDA-core
 * tiles. */
typedef enum fa_b200_variant {
    FA_B200_VARIANT_AUTO    = 0,
    FA_B200_VARIANT_SIMT    = 1,  /* CUDA-core tiles: any D <= 128, all dtypes, fp32 exact */
    FA_B200_VARIANT_TCGEN05 = 2,  /* TMA + tcgen05/TMEM, the fastest backward on offer: where it is
                                     faster (D = 64) ONE kernel produces dK, dV and dQ, summing dQ
                                     tiles into an fp32 buffer with unordered global additions (as the
                                     reference does, kernels/backward_kernel.py:179-194): dQ is then
                                     not bit-reproducible.  Forward: identical to 2PASS.          */
    FA_B200_VARIANT_TCGEN05_2PASS = 3
                                  /* the same family with the two-pass backward (what AUTO runs):
                                     one kernel for dK, dV and one for dQ, every output element
                                     owned by one CTA and summed in a fixed order, so all
                                     gradients are bit-reproducible.                              */
} fa_b200_variant;

/* One (B, N, H, D) tensor: base pointer and element strides (D stride is 1). */
typedef struct fa_b200_tensor {
    void*   ptr;
    int64_t stride_b;
    int64_t stride_n;
    int64_t stride_h;
} fa_b200_tensor;

/*
 * Argument block shared by forward and backward.  Replaces the positional
 * argument list of the reference launchers (kernels/forward_kernel.py:349-385,
 * kernels/backward_kernel.py:279-316).
 */
typedef struct fa_b200_params {
    size_t         struct_bytes;   /* = sizeof(fa_b200_params); checked            */
    fa_b200_tensor q, k, v;        /* inputs                                       */
    fa_b200_tensor o;              /* forward: output; backward: input             */
    fa_b200_tensor d_o;            /* backward input  (grad of o)                  */
    fa_b200_tensor dq, dk, dv;     /* backward outputs                             */
    float*         lse;            /* (B, H, Nq) fp32; fwd output / bwd input      */
    void*          workspace;      /* backward scratch, >= fa_b200_bwd_workspace_bytes */
    size_t         workspace_bytes;
    int32_t*       status_word;    /* optional int32 the kernels set non-zero when a bounded
                                      device-side wait gives up.  Device memory, or pinned
                                      host memory (which the device can write): the library
                                      then reads it, without synchronising, on entry to every
                                      fa_b200_fwd / fa_b200_bwd* call, and a non-zero value
                                      left by an EARLIER call makes the call return
                                      FA_ETIMEOUT (detail in fa_b200_last_error) after
                                      clearing the word, without launching anything     */
    void*          stream;         /* cudaStream_t                                 */
    uint64_t       seed, offset;   /* dropout stream (Philox key / counter word)   */
    int32_t        B, Nq, Nk, H, Hkv, D;
    int32_t        dtype;          /* fa_b200_dtype                                */
    int32_t        causal;         /* key j visible to query i iff j <= i + causal_shift */
    int32_t        variant;        /* fa_b200_variant                              */
    int32_t        device;         /* CUDA ordinal the pointers live on            */
    float          scale;          /* scores = scale * q.k                         */
    float          dropout_p;      /* [0, 1)                                       */
    int32_t        bwd_phases;     /* 0 = whole backward.  Otherwise a bit mask of the
                                      backward's launches to run, for timing one kernel
                                      alone: 1 = preprocess (delta, scaled lse),
                                      2 = dK/dV kernel, 4 = dQ kernel.  Bits 2 and 4 need
                                      a workspace that an earlier call with bit 1 filled. */
    int32_t        causal_shift;   /* >= 0; 0 aligns the mask's diagonal with the top-left corner (the
                                      reference, kernels/forward_kernel.py:179-182), Nk - Nq with the
                                      bottom-right one (the last query sees every key)                */
    /* Additive score bias, scores = scale * q.k + bias (reference kernels/forward_kernel.py:171-176;
       the reference's backward ignores it and returns a zero grad_bias, ops/attention.py:297-301).
       fp32, logical shape (B, H, Nq, Nk): stride_b / stride_h / stride_n are the element strides over
       batch, head and QUERY index, the key index has stride 1; a stride of 0 broadcasts (a key-padding
       mask is (B, 1, 1, Nk): stride_h = stride_n = 0).  -inf entries mask keys.  ptr = NULL: no bias.
       Calls with a bias are served by the CUDA-core kernels. */
    fa_b200_tensor bias;
    /* backward, optional: dense (B, H, Nq, Nk) fp32 buffer, zero-filled by the caller, that receives
       d(loss)/d(scores) = P o (dP o Z - delta); the caller sums it over the bias' broadcast
       dimensions to get grad_bias.  NULL: not produced. */
    float*         d_scores;
    /* Optional per-batch key counts (device pointer to B int32; NULL: every batch entry has Nk keys):
       batch entry b attends to keys [0, kv_lengths[b]) only, the rest of its K/V rows are padding.
       Values are clamped to [1, Nk].  dK and dV rows of the padding are written as zeros.  No counterpart
       in the reference, which expresses padding as a dense -inf bias (examples/basic_usage.py:243-248);
       here whole key blocks beyond the count are skipped, on every kernel family. */
    const int32_t* kv_lengths;
    /* Dropout stream of a call over a slice of a larger problem (a head or batch shard, one chunk of a
       batch).  The mask of column (b, h) is indexed by (b + rng_batch_offset) * rng_heads + h +
       rng_head_offset; rng_heads = 0 means H (the call is the whole problem, offsets then are 0).  A
       sharded or chunked call that passes its slice's origin and the whole problem's head count draws
       exactly the mask the whole call draws.  The reference has no replayable stream at all
       (kernels/forward_kernel.py:198-203). */
    int32_t        rng_batch_offset, rng_head_offset, rng_heads;
    /* Limit of one device-side wait in milliseconds (0: the default, 2000).  A kernel whose wait on an
       mbarrier runs out stops its pipeline, frees what it holds, returns normally and writes a non-zero
       code to *status_word; it never traps and never waits longer. */
    int32_t        wait_limit_ms;
    /* Optional residual of the output, same shape and dtype as o (ptr = NULL: none).  The forward
       writes o_lo = round(O - o), what the rounding of O to 16 bits dropped; the backward, given the
       same tensor, forms delta = rowsum(dO o (o + o_lo)) instead of rowsum(dO o o).  For rows whose
       attention is peaked, dS = P o (dP - delta) cancels nearly equal terms and the bf16 rounding of
       the saved output (2^-9) is the largest error in dQ and dK; with the residual it is gone.  The
       reference saves its output in the tensors' dtype only (ops/attention.py:209-214). */
    fa_b200_tensor o_lo;
    /* Optional buffer for the call's dropout keep bits (NULL: the kernels draw their bits themselves,
       which costs the tensor-core kernels' softmax threads about as many instructions as the attention
       math).  With a buffer of fa_b200_dropout_bits_bytes(&p) bytes (16-byte aligned) a separate kernel
       writes every keep bit of the call once, packed in the two orientations the kernels read (by query
       row for the forward and dQ, by key row for dK/dV), and the tensor-core kernels load them.
       dropout_bits_ready = 0: this call fills the buffer first; 1: the buffer holds the bits an earlier
       call with the same (seed, offset, dropout_p, sizes, causal mask, rng_* origin) wrote, e.g. the
       forward's, and is only read.  Half the size serves a forward alone (no backward follows).  The
       mask is the one fa_b200_dropout_mask_host describes either way.  Ignored without dropout and by
       the CUDA-core kernels. */
    void*          dropout_bits;
    size_t         dropout_bits_bytes;
    int32_t        dropout_bits_ready;
} fa_b200_params;

/* Static tile choice for a (D, dtype, causal) key; replaces the reference's
 * run-time tuner (kernels/autotuning.py:841-952, config.py:288-348). */
typedef struct fa_b200_tile {
    int32_t variant;        /* fa_b200_variant actually used                  */
    int32_t block_m;        /* query rows per tile                            */
    int32_t block_n;        /* key rows per tile                              */
    int32_t q_tiles_per_cta;
    int32_t kv_stages;      /* ring depth: forward K and V tiles; backward, the
                               streamed tile read twice per step (Q_i or K_j)  */
    int32_t num_warps;
    int32_t w_stages;       /* backward: ring depth of the other streamed tile */
    int32_t regs_softmax;   /* forward: registers per softmax thread ...        */
    int32_t regs_other;     /* ... and per MMA / TMA / converting thread        */
    int32_t one_kernel_backward;  /* backward: dK, dV and dQ from one kernel    */
} fa_b200_tile;

/* Forward: o, lse <- attention(q, k, v).  Replaces
 * kernels/forward_kernel.py:246-387 (launcher) and :18-243 (kernel). */
int fa_b200_fwd(const fa_b200_params* p);

/* Backward: dq, dk, dv <- grad(q, k, v, o, lse, dO).  Replaces
 * kernels/backward_kernel.py:208-318 (launcher) and :17-205 (kernel).
 * With variant AUTO, SIMT or TCGEN05_2PASS every gradient element is summed in a fixed order: two
 * runs give bit-identical dq, dk and dv.  Variant TCGEN05 at D = 64 trades that for speed (dq only). */
int fa_b200_bwd(const fa_b200_params* p);

/*
 * Backward that takes no workspace and allocates nothing.  It has no
 * counterpart in the reference.
 *
 * For callers that cannot give the library scratch memory: hosts that own all
 * device memory and offer plugins no allocator, and paths on which cudaMalloc is
 * not allowed.  Same arguments and results as fa_b200_bwd, except that
 * `workspace` and `workspace_bytes` are ignored: the scratch (delta and the
 * scaled log-sum-exp) is an 8 MiB array built into the library's device image,
 * which every GPU that loads the library keeps until the process exits.
 *
 *  - Limit: B * H * (Nq rounded up to 128) <= 1048576 rows, the same for every
 *    kernel family; larger problems return FA_EWORKSPACE (checked before any
 *    other argument) and must use fa_b200_bwd.
 *  - Nq == 0 zero-fills dk and dv, as fa_b200_bwd does (no scratch is touched).
 *  - Tensor-core calls are served by the two-pass backward (the array holds the
 *    per-row vectors only), so dq, dk and dv are bit-reproducible; they equal
 *    fa_b200_bwd's bit for bit when that is asked for the same variant.
 *  - The first call on each device looks the array's device address up
 *    (cudaGetSymbolAddress, with that device current).  Make that first call
 *    outside any stream capture.
 *  - All calls on a device share the one array and it keeps the previous call's
 *    contents.  The kernels overwrite every entry they later read, so nothing
 *    needs clearing, but two calls whose kernels overlap on the GPU (different
 *    streams, no dependency between them) race on it: serialise them.
 */
int fa_b200_bwd_static(const fa_b200_params* p);

/*
 * Running combination of per-block partial results, for sequence-parallel
 * attention (every rank holds a slice of the sequence; key/value blocks travel
 * around a ring; each (query slice, key block) pair is one fa_b200_fwd or
 * fa_b200_bwd call).  No counterpart in the reference: its sequence-parallel
 * strategy is a stub that splits heads instead (interface.py:437-450,
 * config.py:153-157).
 *
 *   lse_acc != NULL (outputs):   lse' = log(e^lse_acc + e^lse_part),
 *       acc <- acc * e^(lse_acc - lse') + part * e^(lse_part - lse'),  lse_acc <- lse'
 *   lse_acc == NULL (gradients): acc <- acc + part
 *
 * acc is (B, N, H, D) fp32, dense within a batch entry (acc_stride_b elements
 * between entries; 0 = N*H*D), lse_acc is (B, H, N) fp32 with strides
 * lse_stride_b / lse_stride_h (0 = dense) and lse_part is dense (B, H, N) fp32
 * (natural log, as fa_b200_fwd writes them): the strides let a call work on a
 * range of rows of a larger total.  `first` != 0: acc and lse_acc
 * hold nothing yet and are overwritten, not read.  out.ptr != NULL: the new
 * total is also written there in `dtype` (the caller sets it on the step it
 * knows to be the last).  part.ptr == NULL with out.ptr != NULL: only that
 * conversion.  D must be a multiple of 8; pointers and strides 16-byte aligned.
 */
typedef struct fa_b200_combine_params {
    size_t         struct_bytes;   /* = sizeof(fa_b200_combine_params); checked */
    float*         acc;
    float*         lse_acc;
    fa_b200_tensor part;           /* (B, N, H, D) in `dtype`, element strides */
    const float*   lse_part;
    fa_b200_tensor out;            /* optional */
    int32_t        B, N, H, D;
    int32_t        dtype;          /* fa_b200_dtype of part and out */
    int32_t        first;
    int32_t        device;
    int32_t        reserved;
    void*          stream;         /* cudaStream_t */
    int64_t        acc_stride_b;   /* elements; 0 = N*H*D */
    int64_t        lse_stride_b;   /* elements of lse_acc; 0 = H*N */
    int64_t        lse_stride_h;   /* 0 = N */
} fa_b200_combine_params;

int fa_b200_combine(const fa_b200_combine_params* p);

/*
 * One strided copy between host and device memory on `stream`: `rows` rows of
 * `row_bytes` bytes, `src_pitch` / `dst_pitch` bytes from one row to the next
 * (cudaMemcpy2DAsync; the direction is inferred from the pointers).  With it a
 * head slice [b, :, h0:h1, :] of a (B, N, H, D) tensor in pinned host memory
 * moves to or from the device in one request: rows of (h1-h0)*D elements, pitch
 * H*D elements.  No counterpart in the reference, whose tensors never leave
 * the device; used by the host-operand pipeline.  Host memory must be pinned
 * for the copy to be asynchronous.
 */
int fa_b200_copy_rows(void* dst, size_t dst_pitch, const void* src, size_t src_pitch,
                      size_t row_bytes, size_t rows, int device, void* stream);

/* Bytes of scratch fa_b200_bwd needs for these sizes (delta, fp32 dQ
 * accumulator, ...).  Counterpart of the 'delta' entry of
 * ops/memory.py:653-760 allocate_attention_workspace_enhanced. */
size_t fa_b200_bwd_workspace_bytes(const fa_b200_params* p);

/* Bytes of fa_b200_params.dropout_bits for this problem (both orientations: B*H * ceil128(Nq) *
 * ceil128(Nk) / 4), or 0 when the call has no dropout or would not be served by the tensor-core
 * kernels.  Pointers in *p may be null.  No counterpart in the reference, which keeps no mask. */
size_t fa_b200_dropout_bits_bytes(const fa_b200_params* p);

/* Tile table lookup; counterpart of config.py:288-348 get_enhanced_config. */
int fa_b200_tile_config(int D, int dtype, int causal, int backward, fa_b200_tile* out);

/*
 * Dropout keep-mask of the kernels' Philox4x32-10 stream, generated on the
 * host: out[((b*H + h)*Nq + i)*Nk + j] = 1 if P[b,h,i,j] is kept, else 0.
 * The reference draws its mask inside the Triton kernel
 * (kernels/forward_kernel.py:198-203) and never replays it; here forward,
 * backward and this function share one integer definition.
 */
int fa_b200_dropout_mask_host(uint64_t seed, uint64_t offset, float dropout_p,
                              int B, int H, int Nq, int Nk, uint8_t* out);

/* Same mask, generated by the device code path the kernels use, written to a
 * device buffer of B*H*Nq*Nk bytes on `stream`. */
int fa_b200_dropout_mask_device(uint64_t seed, uint64_t offset, float dropout_p,
                                int B, int H, int Nq, int Nk, uint8_t* out_dev,
                                int device, void* stream);

/* Drop probability actually realised for a requested dropout_p: the keep test
 * compares one random byte with round(p*256), so p is quantised to 1/256 and
 * kept values are scaled by 1/(1 - effective p). */
float fa_b200_dropout_effective_p(float dropout_p);

/* Raw Philox4x32-10 block (public algorithm, Salmon et al. 2011), exposed so
 * callers can check the generator against its published known answers. */
void fa_b200_philox4x32_10(const uint32_t counter[4], const uint32_t key[2], uint32_t out[4]);

/*
 * Self-test of the bounded device-side wait, the mechanism behind FA_ETIMEOUT: launches one small
 * kernel in which a thread waits, for at most `limit_ms` (1..1000) milliseconds, on an mbarrier that
 * nothing ever arrives at.  The kernel returns normally and writes 9 to *status_word (device memory or
 * pinned host memory).  With a word in pinned host memory the next fa_b200_fwd / fa_b200_bwd call that
 * is given the same word then returns FA_ETIMEOUT.  No counterpart in the reference, whose error path
 * is a Python try/except around the launch (interface.py:331-348).
 */
int fa_b200_selftest_wait_timeout(int32_t* status_word, int limit_ms, int device, void* stream);

const char* fa_b200_strerror(int status);
const char* fa_b200_last_error(void);
int         fa_b200_version(void);

#ifdef __cplusplus
}
#endif
#endif /* FA_B200_H */
