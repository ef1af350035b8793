// C-ABI layer of libfa_b200.so: argument validation, kernel-family choice,
// workspace layout, the static tile table, error strings and the host side of
// the dropout stream.  Everything here is O(1) host work per call: no tensor
// scans and no device synchronisation (the reference's launchers do both:
// utils.py:227-254, kernels/forward_kernel.py:308-313).
#include "fa_common.cuh"
#include "sm100_ptx.cuh"
#include "tile_config.cuh"
#include <stdarg.h>
#include <string.h>
#include <mutex>

namespace fa {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

BwdWorkspace bwd_workspace_layout(const fa_b200_params& p, int variant, bool inline_conversion) {
    BwdWorkspace w;
    memset(&w, 0, sizeof(w));
    const size_t nq_pad = align_up((size_t)p.Nq, 128);
    const bool tc = (variant == FA_B200_VARIANT_TCGEN05 || variant == FA_B200_VARIANT_TCGEN05_2PASS);
    const bool copies = tc && p.dtype == FA_B200_BF16 && !inline_conversion;
    const bool one_kernel = (variant == FA_B200_VARIANT_TCGEN05 && sm100_bwd_fused_supported(p));
    size_t at = 0;
    auto region = [&](size_t* off, size_t* bytes, size_t n) { *off = at; *bytes = n; at = align_up(at + n, 256); };
    const size_t rows = (size_t)p.B * p.H * nq_pad * sizeof(float);
    region(&w.delta_off, &w.delta_bytes, rows);
    region(&w.lse2_off, &w.lse2_bytes, tc ? rows : 0);
    region(&w.rng_off, &w.rng_bytes, tc ? (size_t)p.B * p.Hkv * 2 * sizeof(float) : 0);
    region(&w.erow_off, &w.erow_bytes, copies ? rows : 0);
    region(&w.q16_off, &w.q16_bytes, copies ? (size_t)p.B * p.Nq * p.H * p.D * 2 : 0);
    region(&w.do16_off, &w.do16_bytes, copies ? (size_t)p.B * p.Nq * p.H * p.D * 2 : 0);
    // the K copy feeds the dQ kernel only: the one-kernel backward has none
    region(&w.k16_off, &w.k16_bytes, (copies && !one_kernel) ? (size_t)p.B * p.Nk * p.Hkv * p.D * 2 : 0);
    region(&w.dq_off, &w.dq_bytes, one_kernel ? (size_t)p.B * p.H * nq_pad * (size_t)p.D * sizeof(float) : 0);
    w.total = at ? at : 256;
    return w;
}

int sm_count(int device) {
    static std::mutex mu;
    static int cache[64] = {};
    if (device < 0 || device >= 64) return 0;
    std::lock_guard<std::mutex> lock(mu);
    if (cache[device] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return 0;
        cache[device] = n;
    }
    return cache[device];
}

namespace {

struct GuardDevice {
    int prev = -1;
    bool ok = true;
    explicit GuardDevice(int dev) {
        if (cudaGetDevice(&prev) != cudaSuccess) { ok = false; return; }
        if (prev != dev && cudaSetDevice(dev) != cudaSuccess) ok = false;
    }
    ~GuardDevice() {
        int cur = -1;
        if (prev >= 0 && cudaGetDevice(&cur) == cudaSuccess && cur != prev) cudaSetDevice(prev);
    }
};

int check_tensor(const fa_b200_tensor& t, const char* name, bool required) {
    if (!t.ptr) {
        if (required) { set_error("%s pointer is null", name); return FA_EINVAL; }
        return FA_OK;
    }
    return FA_OK;
}

int validate_common(const fa_b200_params* p, bool backward) {
    if (!p) { set_error("params is null"); return FA_EINVAL; }
    if (p->struct_bytes != sizeof(fa_b200_params)) {
        set_error("struct_bytes %zu does not match this library's fa_b200_params (%zu bytes)",
                  p->struct_bytes, sizeof(fa_b200_params));
        return FA_EINVAL;
    }
    if (p->causal_shift < 0) {
        set_error("causal_shift %d is negative: the first queries would see no key", p->causal_shift);
        return FA_EINVAL;
    }
    if (p->B < 0 || p->Nq < 0 || p->Nk < 0 || p->H <= 0 || p->Hkv <= 0 || p->D <= 0) {
        set_error("sizes must be non-negative and H, Hkv, D positive (B=%d Nq=%d Nk=%d H=%d Hkv=%d D=%d)",
                  p->B, p->Nq, p->Nk, p->H, p->Hkv, p->D);
        return FA_EINVAL;
    }
    if (p->H % p->Hkv != 0) {
        set_error("H (%d) must be a multiple of Hkv (%d)", p->H, p->Hkv);
        return FA_EINVAL;
    }
    if (p->dtype != FA_B200_F16 && p->dtype != FA_B200_BF16 && p->dtype != FA_B200_F32) {
        set_error("unknown dtype %d", p->dtype);
        return FA_EINVAL;
    }
    if (p->variant < FA_B200_VARIANT_AUTO || p->variant > FA_B200_VARIANT_TCGEN05_2PASS) {
        set_error("unknown variant %d", p->variant);
        return FA_EINVAL;
    }
    if (!(p->dropout_p >= 0.f && p->dropout_p < 1.f)) {
        set_error("dropout_p must be in [0, 1), got %g", (double)p->dropout_p);
        return FA_EINVAL;
    }
    if (!(p->scale == p->scale)) { set_error("scale is NaN"); return FA_EINVAL; }
    if (p->rng_batch_offset < 0 || p->rng_head_offset < 0 || p->rng_heads < 0 ||
        (p->rng_heads == 0 && (p->rng_batch_offset || p->rng_head_offset)) ||
        (p->rng_heads > 0 && (int64_t)p->rng_head_offset + p->H > p->rng_heads)) {
        set_error("dropout stream origin (batch %d, head %d of %d heads) does not hold a call with %d heads",
                  p->rng_batch_offset, p->rng_head_offset, p->rng_heads, p->H);
        return FA_EINVAL;
    }
    if (p->wait_limit_ms < 0) { set_error("wait_limit_ms must not be negative"); return FA_EINVAL; }
    if (p->dropout_bits && ((uintptr_t)p->dropout_bits & 15u)) { set_error("dropout_bits must be 16-byte aligned"); return FA_EALIGN; }
    if (p->bwd_phases < 0 || p->bwd_phases > 7) { set_error("bwd_phases must be a mask in [0, 7]"); return FA_EINVAL; }
    if (p->B == 0 || p->Nq == 0) return FA_OK;   // empty problem: nothing else to check
    int rc;
    if ((rc = check_tensor(p->q, "q", true))) return rc;
    if ((rc = check_tensor(p->o, "o", true))) return rc;
    if (p->Nk > 0) {
        if ((rc = check_tensor(p->k, "k", true))) return rc;
        if ((rc = check_tensor(p->v, "v", true))) return rc;
    }
    if (!p->lse) { set_error("lse pointer is null"); return FA_EINVAL; }
    if (backward) {
        if ((rc = check_tensor(p->d_o, "d_o", true))) return rc;
        if ((rc = check_tensor(p->dq, "dq", true))) return rc;
        if (p->Nk > 0) {
            if ((rc = check_tensor(p->dk, "dk", true))) return rc;
            if ((rc = check_tensor(p->dv, "dv", true))) return rc;
        }
    }
    return FA_OK;
}

// A status word in pinned host memory is read here, on entry to the next call, without any
// synchronisation: the kernels write it with a system-wide store when a bounded wait gives up.
// Returns the code an earlier call left (and clears it), 0 when there is none or when the word
// lives in device memory (which only the caller can read, after synchronising).
int take_host_status(int32_t* word) {
    if (!word) return 0;
    static thread_local int32_t* last_word = nullptr;
    static thread_local volatile int32_t* last_host = nullptr;
    if (word != last_word) {
        cudaPointerAttributes attr;
        volatile int32_t* host = nullptr;
        if (cudaPointerGetAttributes(&attr, word) == cudaSuccess && attr.type == cudaMemoryTypeHost)
            host = (volatile int32_t*)attr.hostPointer;
        else
            (void)cudaGetLastError();          // not a CUDA allocation: leave no sticky error behind
        last_word = word;
        last_host = host;
    }
    if (!last_host) return 0;
    const int code = *last_host;
    if (code != 0) *last_host = 0;
    return code;
}

int refuse_after_timeout(const fa_b200_params* p, const char* what) {
    const int code = take_host_status(p->status_word);
    if (code == 0) return FA_OK;
    set_error("%s: an earlier call's device-side wait ran out (status %d: 1 forward, 2 dK/dV, 3 dQ, 4 one-kernel "
              "backward, 5 fp32 forward, 8 shared memory, 9 self-test); its results are invalid.  The word has been cleared", what, code);
    return FA_ETIMEOUT;
}

// Self-test of the bounded wait: one thread waits on an mbarrier that nobody ever arrives at.
__global__ void wait_timeout_selftest_kernel(int32_t* status, int limit_ms) {
    __shared__ uint64_t bar;
    __shared__ uint32_t ctl[2];
    if (threadIdx.x == 0) {
        ptx::mbar_init(&bar, 1u);
        ptx::wait_control_init(ctl, limit_ms);
        ptx::fence_mbar_init();
    }
    __syncthreads();
    if (threadIdx.x == 0 && !ptx::mbar_wait(&bar, 0u, ctl)) ptx::report_status(status, 9);
}

// Kernel family for a call: an explicit request is honoured or refused, AUTO
// prefers the tensor-core family and falls back to CUDA-core tiles for shapes
// it does not cover.
int choose_variant(const fa_b200_params& p, bool backward, int* variant) {
    const char* why = "";
    bool tc = sm100_supports(p, backward, &why);
    if (p.variant == FA_B200_VARIANT_TCGEN05 || p.variant == FA_B200_VARIANT_TCGEN05_2PASS) {
        if (!tc) { set_error("tcgen05 kernels do not cover this call: %s", why); return FA_EUNSUPPORTED; }
        *variant = p.variant;
        return FA_OK;
    }
    // AUTO is the deterministic form: every gradient element is summed by one CTA in a fixed order.
    // The one-kernel backward (dQ tiles summed with unordered global additions) is opt-in (TCGEN05).
    if (p.variant == FA_B200_VARIANT_AUTO && tc) { *variant = FA_B200_VARIANT_TCGEN05_2PASS; return FA_OK; }
    if (!simt_supports(p)) {
        set_error("no kernel covers D=%d (CUDA-core tiles need D <= 128; tensor-core tiles: %s)", p.D, why);
        return FA_EUNSUPPORTED;
    }
    *variant = FA_B200_VARIANT_SIMT;
    return FA_OK;
}

// Zero-fill of dK and dV for a call without queries (shared by both backward entry points).
int zero_dk_dv(const fa_b200_params* p) {
    size_t eb = dtype_bytes(p->dtype);
    for (int b = 0; b < p->B; ++b)
        for (int j = 0; j < p->Nk; ++j) {
            FA_CUDA_CHECK(cudaMemset2DAsync((char*)p->dk.ptr + ((int64_t)b * p->dk.stride_b + (int64_t)j * p->dk.stride_n) * eb,
                                            p->dk.stride_h * eb, 0, p->D * eb, p->Hkv, (cudaStream_t)p->stream));
            FA_CUDA_CHECK(cudaMemset2DAsync((char*)p->dv.ptr + ((int64_t)b * p->dv.stride_b + (int64_t)j * p->dv.stride_n) * eb,
                                            p->dv.stride_h * eb, 0, p->D * eb, p->Hkv, (cudaStream_t)p->stream));
        }
    return FA_OK;
}

}  // namespace
}  // namespace fa

using namespace fa;

extern "C" {

int fa_b200_version(void) { return FA_B200_ABI_VERSION; }

const char* fa_b200_last_error(void) { return g_err; }

const char* fa_b200_strerror(int status) {
    switch (status) {
        case FA_OK:           return "ok";
        case FA_EINVAL:       return "invalid argument";
        case FA_EUNSUPPORTED: return "unsupported shape or dtype";
        case FA_EALIGN:       return "pointer or stride not aligned as the kernel requires";
        case FA_EWORKSPACE:   return "workspace missing or too small";
        case FA_ECUDA:        return "CUDA call failed";
        case FA_ETIMEOUT:     return "a bounded device-side wait of an earlier call ran out";
        default:              return "unknown status";
    }
}

int fa_b200_selftest_wait_timeout(int32_t* status_word, int limit_ms, int device, void* stream) {
    if (!status_word) { set_error("status_word is null"); return FA_EINVAL; }
    if (limit_ms < 1 || limit_ms > 1000) { set_error("limit_ms must be in [1, 1000]"); return FA_EINVAL; }
    GuardDevice g(device);
    if (!g.ok) { set_error("cudaSetDevice(%d) failed", device); return FA_ECUDA; }
    wait_timeout_selftest_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(status_word, limit_ms);
    FA_CUDA_CHECK(cudaGetLastError());
    return FA_OK;
}

int fa_b200_fwd(const fa_b200_params* p) {
    int rc = validate_common(p, false);
    if (rc) return rc;
    if ((rc = refuse_after_timeout(p, "fa_b200_fwd"))) return rc;
    if (p->B == 0 || p->Nq == 0) return FA_OK;
    if (p->Nk == 0) { set_error("Nk = 0: softmax over an empty key set is undefined"); return FA_EINVAL; }
    int variant;
    if ((rc = choose_variant(*p, false, &variant))) return rc;
    GuardDevice g(p->device);
    if (!g.ok) { set_error("cudaSetDevice(%d) failed", p->device); return FA_ECUDA; }
    return variant != FA_B200_VARIANT_SIMT ? sm100_fwd(*p) : simt_fwd(*p);
}

int fa_b200_copy_rows(void* dst, size_t dst_pitch, const void* src, size_t src_pitch,
                      size_t row_bytes, size_t rows, int device, void* stream) {
    if (row_bytes == 0 || rows == 0) return FA_OK;
    if (!dst || !src) { set_error("copy_rows: null pointer"); return FA_EINVAL; }
    if (dst_pitch < row_bytes || src_pitch < row_bytes) {
        set_error("copy_rows: pitch (%zu, %zu) smaller than the row (%zu bytes)", dst_pitch, src_pitch, row_bytes);
        return FA_EINVAL;
    }
    GuardDevice g(device);
    if (!g.ok) { set_error("cudaSetDevice(%d) failed", device); return FA_ECUDA; }
    if (dst_pitch == row_bytes && src_pitch == row_bytes)
        FA_CUDA_CHECK(cudaMemcpyAsync(dst, src, row_bytes * rows, cudaMemcpyDefault, (cudaStream_t)stream));
    else
        FA_CUDA_CHECK(cudaMemcpy2DAsync(dst, dst_pitch, src, src_pitch, row_bytes, rows, cudaMemcpyDefault,
                                        (cudaStream_t)stream));
    return FA_OK;
}

size_t fa_b200_bwd_workspace_bytes(const fa_b200_params* p) {
    if (!p || p->struct_bytes != sizeof(fa_b200_params)) return 0;
    if (p->B <= 0 || p->Nq <= 0 || p->H <= 0 || p->Hkv <= 0 || p->D <= 0) return 256;
    int variant = FA_B200_VARIANT_SIMT;
    fa_b200_params q = *p;
    // Size for the largest family the call could be routed to, so that the
    // answer does not depend on pointer alignment (pointers may be null here).
    const char* why = "";
    q.variant = FA_B200_VARIANT_AUTO;
    if (p->variant != FA_B200_VARIANT_SIMT && sm100_supports(q, true, &why))
        variant = (p->variant == FA_B200_VARIANT_TCGEN05) ? FA_B200_VARIANT_TCGEN05 : FA_B200_VARIANT_TCGEN05_2PASS;
    return bwd_workspace_layout(*p, variant).total;
}

size_t fa_b200_dropout_bits_bytes(const fa_b200_params* p) {
    if (!p || p->struct_bytes != sizeof(fa_b200_params)) return 0;
    if (p->B <= 0 || p->Nq <= 0 || p->Nk <= 0 || p->H <= 0 || p->Hkv <= 0 || p->D <= 0) return 0;
    if (dropout_threshold(p->dropout_p) == 0u || p->variant == FA_B200_VARIANT_SIMT) return 0;
    fa_b200_params q = *p;
    q.variant = FA_B200_VARIANT_AUTO;
    const char* why = "";
    if (!sm100_supports(q, false, &why) && !sm100_supports(q, true, &why)) return 0;
    return 2 * dropout_bits_bytes(*p);
}

int fa_b200_bwd(const fa_b200_params* p) {
    int rc = validate_common(p, true);
    if (rc) return rc;
    if ((rc = refuse_after_timeout(p, "fa_b200_bwd"))) return rc;
    if (p->B == 0 || (p->Nq == 0 && p->Nk == 0)) return FA_OK;
    if (p->Nk == 0) { set_error("Nk = 0: softmax over an empty key set is undefined"); return FA_EINVAL; }
    int variant;
    if ((rc = choose_variant(*p, true, &variant))) return rc;
    BwdWorkspace ws = bwd_workspace_layout(*p, variant);
    if (!p->workspace || p->workspace_bytes < ws.total) {
        set_error("backward needs %zu bytes of workspace, got %zu", ws.total,
                  p->workspace ? p->workspace_bytes : (size_t)0);
        return FA_EWORKSPACE;
    }
    if (((uintptr_t)p->workspace & 255u) != 0) {
        set_error("workspace must be 256-byte aligned");
        return FA_EALIGN;
    }
    GuardDevice g(p->device);
    if (!g.ok) { set_error("cudaSetDevice(%d) failed", p->device); return FA_ECUDA; }
    if (p->Nq == 0) return zero_dk_dv(p);      // no queries: dK = dV = 0
    return variant != FA_B200_VARIANT_SIMT ? sm100_bwd(*p, ws) : simt_bwd(*p, ws);
}

// ---------------------------------------------------------------------------
// Backward without a caller-supplied workspace.
//
// Some hosts of this library cannot hand it scratch memory: a runtime that owns
// all device memory itself and exposes no allocator to plugins, or a caller on a
// path where cudaMalloc is forbidden (inside a latency-critical loop, under a
// memory budget fixed at start-up).  For them the backward's scratch (delta and
// the scaled log-sum-exp, 8 bytes per padded query row) lives in a fixed array
// in the library's own device image.  Every GPU that loads the library holds
// these bytes until the process exits.
constexpr uint64_t kStaticScratchRows = 1u << 20;         // B * H * ceil128(Nq) a call may have
// two fp32 vectors of that many rows (8 MiB) + the per-column ranges (at most rows / 128 columns) + alignment
constexpr size_t kStaticScratchBytes = (8u << 20) + (kStaticScratchRows / 128) * 8 + 512;
static __device__ __align__(256) unsigned char g_bwd_static_scratch[kStaticScratchBytes];

namespace {
constexpr int kMaxDevices = 64;
std::mutex g_scratch_mutex;
void* g_scratch_ptr[kMaxDevices] = {};

// Device address of the array on the CURRENT device.  In host code the array's
// name is only a handle; the address kernels can use comes from
// cudaGetSymbolAddress, asked once per device with that device current.
int static_scratch_address(int device, void** out) {
    if (device < 0 || device >= kMaxDevices) { set_error("device %d out of range", device); return FA_EINVAL; }
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    if (!g_scratch_ptr[device]) {
        void* ptr = nullptr;
        FA_CUDA_CHECK(cudaGetSymbolAddress(&ptr, g_bwd_static_scratch));
        g_scratch_ptr[device] = ptr;
    }
    *out = g_scratch_ptr[device];
    return FA_OK;
}
}  // namespace

int fa_b200_bwd_static(const fa_b200_params* p) {
    // The size limit comes before everything else, pointers included: it needs the sizes only, and a
    // call beyond it never gets near a launch whatever its other arguments are.  One limit for every
    // kernel family (the CUDA-core family would fit twice as many rows; it is held to the same number).
    if (p && p->struct_bytes == sizeof(fa_b200_params) && p->B > 0 && p->H > 0 && p->Nq > 0) {
        const uint64_t rows = (uint64_t)p->B * (uint64_t)p->H * (uint64_t)align_up((size_t)p->Nq, 128);
        if (rows > kStaticScratchRows) {
            set_error("fa_b200_bwd_static: B*H*(Nq rounded up to 128) = %llu rows, the built-in array serves at most "
                      "%llu (1048576); use fa_b200_bwd with a workspace",
                      (unsigned long long)rows, (unsigned long long)kStaticScratchRows);
            return FA_EWORKSPACE;
        }
    }
    int rc = validate_common(p, true);
    if (rc) return rc;
    if ((rc = refuse_after_timeout(p, "fa_b200_bwd_static"))) return rc;
    if (p->B == 0 || (p->Nq == 0 && p->Nk == 0)) return FA_OK;
    if (p->Nk == 0) { set_error("Nk = 0: softmax over an empty key set is undefined"); return FA_EINVAL; }
    int variant;
    if ((rc = choose_variant(*p, true, &variant))) return rc;
    // the built-in array is sized for the per-row vectors only: tensor-core calls take the two-pass backward
    if (variant == FA_B200_VARIANT_TCGEN05) variant = FA_B200_VARIANT_TCGEN05_2PASS;
    BwdWorkspace ws = bwd_workspace_layout(*p, variant, /*inline_conversion=*/true);
    if (ws.total > kStaticScratchBytes) {
        set_error("fa_b200_bwd_static: this problem needs %zu bytes of scratch, the built-in array holds %zu; "
                  "use fa_b200_bwd with a workspace", ws.total, kStaticScratchBytes);
        return FA_EWORKSPACE;
    }
    GuardDevice g(p->device);
    if (!g.ok) { set_error("cudaSetDevice(%d) failed", p->device); return FA_ECUDA; }
    if (p->Nq == 0) return zero_dk_dv(p);      // no queries: dK = dV = 0, as fa_b200_bwd does; needs no scratch
    void* scratch = nullptr;
    if ((rc = static_scratch_address(p->device, &scratch))) return rc;
    fa_b200_params q = *p;
    q.workspace = scratch;
    q.workspace_bytes = kStaticScratchBytes;
    // Nothing in the scratch has to start at zero: the preprocess launch writes
    // every delta / lse entry (padding included) before the main kernels read them.
    return variant != FA_B200_VARIANT_SIMT ? sm100_bwd(q, ws) : simt_bwd(q, ws);
}

// Static tile table.  Tensor-core rows report the constants the sm_100a kernels are compiled from
// (tile_config.cuh); everything else is served by 64x64 CUDA-core tiles.  The same tiles serve both
// masks: `causal` is part of the reference's lookup key (config.py:288-348) and changes no row here.
int fa_b200_tile_config(int D, int dtype, int causal, int backward, fa_b200_tile* out) {
    if (!out) { set_error("out is null"); return FA_EINVAL; }
    if (D <= 0 || D > 128) { set_error("no tile for D=%d", D); return FA_EUNSUPPORTED; }
    (void)causal;
    memset(out, 0, sizeof(*out));
    bool tc = (dtype == FA_B200_F16 || dtype == FA_B200_BF16) && (D == 64 || D == 128);
    if (tc) {
        out->variant = FA_B200_VARIANT_TCGEN05_2PASS;     // what AUTO runs
        out->block_m = tile::kBlockM;
        out->block_n = tile::kBlockN;
        out->q_tiles_per_cta = backward ? 1 : tile::kFwdQTilesPerCta;
        out->kv_stages = backward ? tile::bwd_u_stages(D, false) : tile::fwd_kv_stages(D);
        out->w_stages = backward ? tile::bwd_w_stages(D) : 0;
        out->num_warps = backward ? tile::kBwdWarps : tile::kFwdWarps;
        out->regs_softmax = backward ? 0 : tile::kFwdRegsSoftmax;
        out->regs_other = backward ? 0 : tile::kFwdRegsOther;
        out->one_kernel_backward = backward && tile::bwd_one_kernel(D) ? 1 : 0;   // available on request (TCGEN05)
    } else {
        out->variant = FA_B200_VARIANT_SIMT;
        out->block_m = 64;
        out->block_n = 64;
        out->q_tiles_per_cta = 1;
        out->kv_stages = 1;
        out->num_warps = 8;
    }
    return FA_OK;
}

void fa_b200_philox4x32_10(const uint32_t counter[4], const uint32_t key[2], uint32_t out[4]) {
    philox4x32_10(counter[0], counter[1], counter[2], counter[3], key[0], key[1], out);
}

float fa_b200_dropout_effective_p(float dropout_p) { return dropout_effective_p(dropout_p); }

int fa_b200_dropout_mask_host(uint64_t seed, uint64_t offset, float dropout_p,
                              int B, int H, int Nq, int Nk, uint8_t* out) {
    if (B < 0 || H < 0 || Nq < 0 || Nk < 0) { set_error("negative size"); return FA_EINVAL; }
    if ((int64_t)B * H * Nq * Nk == 0) return FA_OK;
    if (!out) { set_error("out is null"); return FA_EINVAL; }
    if (!(dropout_p >= 0.f && dropout_p < 1.f)) { set_error("dropout_p must be in [0, 1)"); return FA_EINVAL; }
    PhiloxKey key = philox_make_key(seed, offset);
    uint32_t thr = dropout_threshold(dropout_p);
    int jb_per_row = (Nk + 15) / 16;
    for (int64_t rowid = 0; rowid < (int64_t)B * H * Nq; ++rowid) {
        uint32_t bh = (uint32_t)(rowid / Nq), i = (uint32_t)(rowid % Nq);
        uint8_t* dst = out + rowid * Nk;
        for (int jb = 0; jb < jb_per_row; ++jb) {
            uint32_t bits = thr ? dropout_keep_bits(key, bh, i, (uint32_t)jb, thr) : 0xFFFFu;
            for (int c = 0; c < 16 && jb * 16 + c < Nk; ++c) dst[jb * 16 + c] = (bits >> c) & 1u;
        }
    }
    return FA_OK;
}

int fa_b200_dropout_mask_device(uint64_t seed, uint64_t offset, float dropout_p,
                                int B, int H, int Nq, int Nk, uint8_t* out_dev,
                                int device, void* stream) {
    if (B < 0 || H < 0 || Nq < 0 || Nk < 0) { set_error("negative size"); return FA_EINVAL; }
    if ((int64_t)B * H * Nq * Nk == 0) return FA_OK;
    if (!out_dev) { set_error("out_dev is null"); return FA_EINVAL; }
    if (!(dropout_p >= 0.f && dropout_p < 1.f)) { set_error("dropout_p must be in [0, 1)"); return FA_EINVAL; }
    GuardDevice g(device);
    if (!g.ok) { set_error("cudaSetDevice(%d) failed", device); return FA_ECUDA; }
    return launch_dropout_mask(seed, offset, dropout_p, B, H, Nq, Nk, out_dev, (cudaStream_t)stream);
}

}  // extern "C"
