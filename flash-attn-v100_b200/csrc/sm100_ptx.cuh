// Thin inline-PTX wrappers for the sm_100a features the tensor-core kernels
// use: mbarrier, TMA tensor copies, tcgen05 (TMEM allocation, MMA, commit,
// load/store) and the shared-memory / instruction descriptors of tcgen05.mma.
//
// Every wait is bounded: it gives up after a wall-clock limit, raises the CTA's
// abort flag, and returns false so the caller can unwind (free TMEM, exit).
#pragma once
#include <cuda.h>      // CUtensorMap (type only; the driver entry point is fetched at run time)
#include <stdint.h>

namespace fa {
namespace ptx {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ uint64_t globaltimer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "elect.sync _|p, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(pred));
    return pred != 0;
}

// ---- mbarrier ---------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Warp-aggregated arrive: every lane has finished its part (and issued whatever
// fence its accesses need); one lane arrives for the warp, so a barrier shared by
// W warps is initialised with count W instead of 32 W serialised arrivals.
__device__ __forceinline__ void mbar_arrive_warp(uint64_t* bar) {
    __syncwarp();
    if ((threadIdx.x & 31u) == 0u) mbar_arrive(bar);
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Wall-clock limit of one wait.  The longest legitimate wait inside a CTA is
// one pipeline step (microseconds); the default of two seconds means a protocol
// error.  The caller may pass a shorter one (fa_b200_params.wait_limit_ms).
constexpr uint32_t kDefaultWaitLimitUs = 2000000u;

// The CTA's wait control block in shared memory: word 0 is the abort flag any
// thread may raise (a raised flag ends every wait), word 1 the limit of one wait
// in microseconds.
__device__ __forceinline__ void wait_control_init(volatile uint32_t* abort_flag, int limit_ms) {
    abort_flag[0] = 0u;
    abort_flag[1] = limit_ms > 0 ? (uint32_t)limit_ms * 1000u : kDefaultWaitLimitUs;
}

// Set the caller's status word (device memory, or pinned host memory the host reads without
// synchronising): a plain store made visible system-wide; nothing is read back.
__device__ __forceinline__ void report_status(int32_t* status, int32_t code) {
    if (status) {
        *reinterpret_cast<volatile int32_t*>(status) = code;
        __threadfence_system();
    }
}

// Wait for the phase with the given parity; false when the wait ran out or the flag was raised.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag) {
    if (mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = globaltimer_ns();
    uint32_t spins = 0;
    while (true) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((++spins & 63u) == 0) {
            if (abort_flag[0]) return false;
            if (globaltimer_ns() - t0 > (uint64_t)abort_flag[1] * 1000ull) {
                abort_flag[0] = 1u;
                return false;
            }
        }
    }
}

// ---- proxies / fences ---------------------------------------------------------
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---- global reductions ---------------------------------------------------------
// Four fp32 additions to 16 consecutive bytes of global memory in one request (no return value).
__device__ __forceinline__ void red_add_v4_f32(float* gptr, float x, float y, float z, float w) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};"
                 ::"l"(gptr), "f"(x), "f"(y), "f"(z), "f"(w) : "memory");
}

// ---- TMA ----------------------------------------------------------------------
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* m) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}

// 4-D tiled load global -> shared, completion counted on `bar`; a plain per-CTA load.
__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* map, uint64_t* bar,
                                            int c0, int c1, int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)),
          "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}

// 4-D tiled store shared -> global (bulk async group).
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* map, const void* smem_src,
                                             int c0, int c1, int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
        ::"l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(smem_src)),
          "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void tma_store_wait_all() {
    asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// ---- tcgen05: tensor memory ------------------------------------------------------
// Allocate `ncols` (power of two, 32..512) TMEM columns; one full warp calls
// this; the base address is written to *smem_out.
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_out, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(smem_out)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ---- tcgen05: MMA -----------------------------------------------------------------
// D[tmem] (+)= A[smem desc] * B[smem desc]; one thread issues.
__device__ __forceinline__ void mma_ss_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                           uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem desc]
__device__ __forceinline__ void mma_ts_f16(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
                                           uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Arrive on `bar` once every MMA this thread issued so far has completed.
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                 ::"r"(smem_u32(bar)) : "memory");
}

// Instruction descriptor of tcgen05.mma kind::f16 (dense, fp32 accumulate).
//   bits 4-5 D format (1 = f32) | 7-9 A format | 10-12 B format (0 = f16, 1 = bf16)
//   bit 15 A major | bit 16 B major (0 = K-major, 1 = MN-major)
//   bits 17-22 N >> 3 | bits 24-28 M >> 4
// A and B carry their own format fields: an fp16 A may meet a bf16 B.
__host__ __device__ constexpr uint32_t make_idesc_f16(bool a_bf16, bool b_bf16, int M, int N, bool a_mn_major,
                                                      bool b_mn_major) {
    return (1u << 4) | ((a_bf16 ? 1u : 0u) << 7) | ((b_bf16 ? 1u : 0u) << 10) |
           ((a_mn_major ? 1u : 0u) << 15) | ((b_mn_major ? 1u : 0u) << 16) |
           ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

// Shared-memory matrix descriptor, 128-byte swizzle (rows of 128 bytes, 8-row
// groups of 1024 bytes, as a TMA box with SWIZZLE_128B lays them out).
//   bits 0-13 start >> 4 | 16-29 leading byte offset >> 4 | 32-45 stride byte
//   offset >> 4 | bits 46-47 = 1 (sm_100 descriptor) | bits 61-63 = 2 (128B swizzle)
// K-major operand:  stride = 1024 (next 8 rows); leading offset unused.
// MN-major operand: stride = 1024 (next 8 K rows); leading = bytes to the next
//                   64-element chunk along M/N.
// `layout`: bits 61-63, 2 = 128-byte swizzle in 16-byte pieces; 1 = 128-byte swizzle in 32-byte
// pieces (the only arrangement of an MN-major 32-bit operand: rows of 128 bytes, 4-row groups of
// 512 bytes; stride = bytes to the next 4 K rows).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr, uint32_t leading_bytes,
                                                   uint32_t stride_bytes, uint32_t layout) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)((leading_bytes >> 4) & 0x3FFFu) << 16;
    d |= (uint64_t)((stride_bytes >> 4) & 0x3FFFu) << 32;
    d |= 1ull << 46;
    d |= (uint64_t)layout << 61;
    return d;
}
__device__ __forceinline__ uint64_t make_smem_desc_sw128(uint32_t smem_addr, uint32_t leading_bytes,
                                                         uint32_t stride_bytes) {
    return make_smem_desc(smem_addr, leading_bytes, stride_bytes, 2u);
}

// ---- tcgen05: TMEM <-> registers ---------------------------------------------------
// 32 lanes x 32 columns of 32 bits: thread t of the warp gets lane (base lane + t),
// r[c] = column (base column + c).  The warp may only touch lanes
// 32*(warp_id % 4) .. +31.
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr),
          "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
// 16 lanes x 256 bits, four times along the columns (32 columns in all): the accumulator-fragment
// layout.  Thread t gets, for j = 0..3:  r[4j], r[4j+1] = lane t/4, columns 8j + 2(t%4), +1;
// r[4j+2], r[4j+3] = lane t/4 + 8, the same columns.  The lane field of taddr picks the 16-lane half.
__device__ __forceinline__ void tmem_ld_16x256b_x4(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.16x256b.x4.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
}
// 16 lanes x 128 bits, twice along the columns (8 columns): thread t holds, for j = 0, 1:
// r[2j] = lane t/4, column 4j + t%4;  r[2j+1] = lane t/4 + 8, the same column.
__device__ __forceinline__ void tmem_st_16x128b_x2(uint32_t taddr, const uint32_t (&r)[4]) {
    asm volatile("tcgen05.st.sync.aligned.16x128b.x2.b32 [%0], {%1, %2, %3, %4};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]) : "memory");
}
__device__ __forceinline__ void tmem_st_32x8(uint32_t taddr, const uint32_t (&r)[8]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
        : "memory");
}
__device__ __forceinline__ void tmem_st_32x16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr),
          "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// ---- small math helpers ----------------------------------------------------------------
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// ---- packed fp32 pairs (sm_100: fma/add/mul on two floats per instruction) -------------
__device__ __forceinline__ uint64_t f2_pack(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void f2_unpack(uint64_t v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t f2_fma(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t f2_add(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ uint64_t f2_mul(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// 2^x for two values on the FMA pipes instead of the 16-lane/clk special-function
// unit: n = round(x) through the 1.5*2^23 magic add, f = x - n in [-0.5, 0.5],
// 2^f by a degree-3 minimax polynomial (relative error 7.5e-5, below the rounding
// of a 16-bit P), and n added into the exponent field.  x is clamped at -126, so
// -inf (masked) gives ~1e-38 instead of 0, which vanishes in every later sum.
__device__ __forceinline__ void ex2_poly2(float x0, float x1, float& p0, float& p1) {
    const uint64_t kMagic = 0x4B4000004B400000ull;      // {12582912.f, 12582912.f}
    const uint64_t kMinus1 = 0xBF800000BF800000ull;     // {-1.f, -1.f}
    const uint64_t kC0 = 0x3F7FFB493F7FFB49ull;         // 0.99992806
    const uint64_t kC1 = 0x3F31798D3F31798Dull;         // 0.69326097
    const uint64_t kC2 = 0x3E786F0D3E786F0Dull;         // 0.24261113
    const uint64_t kC3 = 0x3D61FBB03D61FBB0ull;         // 0.05517167
    const uint64_t x = f2_pack(fmaxf(x0, -126.f), fmaxf(x1, -126.f));
    const uint64_t t = f2_add(x, kMagic);
    const uint64_t neg_n = f2_fma(t, kMinus1, kMagic);
    const uint64_t f = f2_add(x, neg_n);
    uint64_t r = f2_fma(f, kC3, kC2);
    r = f2_fma(r, f, kC1);
    r = f2_fma(r, f, kC0);
    float r0, r1, t0, t1;
    f2_unpack(r, r0, r1);
    f2_unpack(t, t0, t1);
    p0 = __uint_as_float(__float_as_uint(r0) + (__float_as_uint(t0) << 23));
    p1 = __uint_as_float(__float_as_uint(r1) + (__float_as_uint(t1) << 23));
}

// two floats -> packed 16-bit pair; `lo` lands in bits 0-15
template <bool BF16>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    uint32_t r;
    if (BF16) asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    else      asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

// ---- bf16 -> fp16 in shared memory ---------------------------------------------------------------
// tcgen05.mma kind::f16 wants both operands in one 16-bit format.  A product whose A operand is a
// probability (or dS) tile rounded to bf16 carries that rounding, 2^-9 relative, into the result
// at full size, because with zero-mean V / K / Q / dO the terms add like a random walk; rounded
// to fp16 (2^-12) it does not.  So for bf16 inputs the B operand tile is converted in place, as it
// sits in shared memory after the TMA load, and the MMA runs f16 x f16.  The conversion is exact
// for 2^-17 <= |x| < 65520 (bf16 has 8 significant bits, fp16 11; below 2^-14 fp16 is subnormal
// with a spacing of 2^-24), it saturates beyond and loses bits below; `mul` (a power of two) moves
// a tensor whose values lie elsewhere into that range first.
__device__ __forceinline__ uint32_t bf16x2_to_f16x2(uint32_t x) {
    uint32_t r;
    asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;"
        : "=r"(r) : "f"(__uint_as_float(x & 0xFFFF0000u)), "f"(__uint_as_float(x << 16)));
    return r;
}
__device__ __forceinline__ uint32_t bf16x2_to_f16x2(uint32_t x, uint64_t mul2) {
    float lo, hi;
    f2_unpack(f2_mul(f2_pack(__uint_as_float(x << 16), __uint_as_float(x & 0xFFFF0000u)), mul2), lo, hi);
    uint32_t r;
    asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
// Convert `bytes` (a multiple of 16 * nthreads * 4) of bf16 at `tile` to fp16 in place; thread `t` of
// `nthreads` takes 16-byte pieces t, t + nthreads, ...  Element-wise, so the tile's swizzle is irrelevant.
template <bool SCALED>
__device__ __forceinline__ void convert_tile_bf16_to_f16(uint8_t* tile, int bytes, int t, int nthreads, float mul) {
    uint4* p = reinterpret_cast<uint4*>(tile) + t;
    const uint64_t m2 = f2_pack(mul, mul);
    const int n = bytes / (16 * nthreads);
#pragma unroll 4
    for (int i = 0; i < n; ++i) {
        uint4 v = p[i * nthreads];
        if (SCALED) {
            v.x = bf16x2_to_f16x2(v.x, m2); v.y = bf16x2_to_f16x2(v.y, m2);
            v.z = bf16x2_to_f16x2(v.z, m2); v.w = bf16x2_to_f16x2(v.w, m2);
        } else {
            v.x = bf16x2_to_f16x2(v.x); v.y = bf16x2_to_f16x2(v.y);
            v.z = bf16x2_to_f16x2(v.z); v.w = bf16x2_to_f16x2(v.w);
        }
        p[i * nthreads] = v;
    }
}

// packed 16-bit pair -> two floats (`lo` from bits 0-15)
template <bool BF16>
__device__ __forceinline__ void unpack2(uint32_t v, float& lo, float& hi) {
    if (BF16) {
        lo = __uint_as_float(v << 16);
        hi = __uint_as_float(v & 0xFFFF0000u);
    } else {
        asm("{\n\t.reg .b16 l, h;\n\tmov.b32 {l, h}, %2;\n\tcvt.f32.f16 %0, l;\n\tcvt.f32.f16 %1, h;\n\t}"
            : "=f"(lo), "=f"(hi) : "r"(v));
    }
}

// Programmatic dependent launch.  launch_dependents: the next kernel in the stream, if it was launched
// with programmatic stream serialization, may start once every CTA of this grid has got here (or left).
// dependency_wait: returns when the grids this one was serialized behind have completed and their
// writes are visible.  Both do nothing in a launch without the attribute.
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

}  // namespace ptx
}  // namespace fa
