// Shared device helpers: MX codecs (bit-exact with the CPU oracle) and thin
// wrappers over the sm_100a PTX the kernels use (mbarrier, TMA, tcgen05/TMEM).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#define RK_DEVINL __device__ __forceinline__

namespace rk {

// ----------------------------------------------------------------------------
// Element formats: {ebits, mbits, bias, unbiased emax, max mantissa, fp32
// mantissa of the largest finite value}.  Same table as the CPU oracle.
// ----------------------------------------------------------------------------
struct FmtDesc { int ebits, mbits, bias, emax, max_mant; uint32_t thresh; float fmax; };

template <int FMT> struct FmtT;
template <> struct FmtT<0> { static constexpr int ebits = 4, mbits = 3, bias = 7,  emax = 8,  max_mant = 6; static constexpr uint32_t thresh = 0x600000u; };
template <> struct FmtT<1> { static constexpr int ebits = 5, mbits = 2, bias = 15, emax = 15, max_mant = 3; static constexpr uint32_t thresh = 0x600000u; };
template <> struct FmtT<2> { static constexpr int ebits = 2, mbits = 3, bias = 1,  emax = 2,  max_mant = 7; static constexpr uint32_t thresh = 0x700000u; };
template <> struct FmtT<3> { static constexpr int ebits = 3, mbits = 2, bias = 3,  emax = 4,  max_mant = 3; static constexpr uint32_t thresh = 0x600000u; };
// E2M1 (FP4; lib/golden/mx_fp_math.h:238-246 fp4_e2m1_decode): 0, 0.5, 1, 1.5, 2, 3, 4, 6
template <> struct FmtT<4> { static constexpr int ebits = 2, mbits = 1, bias = 1,  emax = 2,  max_mant = 1; static constexpr uint32_t thresh = 0x400000u; };

template <int FMT> RK_DEVINL float fmt_max() {
  using F = FmtT<FMT>;
  // (1 + max_mant/2^mbits) * 2^emax as an fp32 bit pattern
  return __uint_as_float(((uint32_t)(F::emax + 127) << 23) | ((uint32_t)F::max_mant << (23 - F::mbits)));
}

// round-half-to-even of v >> sh (sh >= 1; sh >= 32 gives 0), the integer
// rounding of kernels/simt_quant/kernel.cpp:44-54.
RK_DEVINL uint32_t round_shift(uint32_t v, int sh) {
  if (sh >= 32) return 0u;
  const uint32_t low = v & ((1u << sh) - 1u), half = 1u << (sh - 1);
  uint32_t q = v >> sh;
  q += (low > half || (low == half && (q & 1u))) ? 1u : 0u;
  return q;
}

// fp32 -> element code, RNE, saturating; kernels/simt_quant/kernel.cpp:56-81
// generalised over the format widths.
template <int FMT> RK_DEVINL uint32_t encode_rne(float xf) {
  using F = FmtT<FMT>;
  constexpr int nb = 1 + F::ebits + F::mbits;
  constexpr uint32_t one = 1u << F::mbits;
  constexpr uint32_t sat = (uint32_t)(((F::emax + F::bias) << F::mbits) | F::max_mant);
  constexpr int emin = 1 - F::bias;
  const uint32_t x = __float_as_uint(xf);
  const uint32_t absx = x & 0x7FFFFFFFu;
  const uint32_t s = (x >> 31) << (nb - 1);
  if (absx == 0u) return s;
  if (__uint_as_float(absx) >= fmt_max<FMT>()) return s | sat;
  const int e = (int)(absx >> 23) - 127;
  const uint32_t sig = (1u << 23) | (absx & 0x7FFFFFu);
  uint32_t out;
  if (e < emin) {
    const uint32_t q = round_shift(sig, (23 - F::mbits) + (emin - e));
    out = q;   // q >= one encodes the smallest normal: (1<<mbits)|(q-one) == q
  } else {
    uint32_t r = round_shift(sig, 23 - F::mbits);
    int E = e;
    if (r == 2 * one) { r = one; E += 1; }
    const int expf = E + F::bias;
    const uint32_t mant = r - one;
    constexpr int expf_max = F::emax + F::bias;
    if (expf > expf_max || (expf == expf_max && (int)mant > F::max_mant)) return s | sat;
    out = ((uint32_t)expf << F::mbits) | mant;
  }
  return s | out;
}

// Block scale of the lib/golden rule from the fp32 bits of amax (amax > 0):
// e = ceil(log2(amax / FMT_MAX)); returns e, the clamped E8M0 code and 2^-e.
template <int FMT> RK_DEVINL void block_scale(float amax, uint32_t& code, float& pow2_neg_e) {
  using F = FmtT<FMT>;
  const uint32_t ab = __float_as_uint(amax);
  const int e = ((int)((ab >> 23) & 0xFFu) - 127 - F::emax) + ((ab & 0x7FFFFFu) > F::thresh ? 1 : 0);
  int sc = e + 127;
  sc = sc < 0 ? 0 : (sc > 254 ? 254 : sc);
  code = (uint32_t)sc;
  pow2_neg_e = __uint_as_float((uint32_t)(127 - e) << 23);
}

// Exact decode of an element code to fp32.
template <int FMT> RK_DEVINL float decode_elem(uint32_t code) {
  using F = FmtT<FMT>;
  constexpr int nb = 1 + F::ebits + F::mbits;
  const uint32_t s = (code >> (nb - 1)) & 1u;
  const uint32_t e = (code >> F::mbits) & ((1u << F::ebits) - 1u);
  const uint32_t m = code & ((1u << F::mbits) - 1u);
  float v;
  if (e == 0) v = (float)m * __uint_as_float((uint32_t)(127 + 1 - F::bias - F::mbits) << 23);
  else v = __uint_as_float(((e + 127 - F::bias) << 23) | (m << (23 - F::mbits)));
  return s ? -v : v;
}

// E8M0 -> fp32 (code 0 = 2^-127 is an fp32 denormal; 0xFF must not be passed).
RK_DEVINL float e8m0_to_f32(uint32_t c) { return __uint_as_float(c == 0 ? 0x00400000u : (c << 23)); }

// ----------------------------------------------------------------------------
// PTX wrappers
// ----------------------------------------------------------------------------
RK_DEVINL uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

RK_DEVINL void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
RK_DEVINL void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
RK_DEVINL void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// One poll of an mbarrier phase.  HINT_NS > 0 lets the hardware keep the thread suspended for up to that many
// ns before it reports "not yet": a warp that waits long (a TMA producer) then issues few instructions and
// leaves the issue slots of its scheduler to the working warps; 0 = the hardware default, quickest wake-up.
template <uint32_t HINT_NS = 0>
RK_DEVINL bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  if (HINT_NS > 0) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity), "r"(HINT_NS) : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  }
  return ok != 0;
}
// Non-blocking test of an mbarrier phase (never suspends the thread): for a look ahead whose answer is used later.
RK_DEVINL bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
RK_DEVINL uint64_t global_timer_ns() {
  uint64_t t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t;
}
// Bounded wait: gives up after about `limit_ns` of wall time (or as soon as this
// CTA's abort flag or the device status word is set by someone else), records
// `code` in *status and returns false; the caller then skips its work so the
// kernel drains and exits instead of hanging the GPU.
// (Measured: a tighter five-instruction polling loop is slower, prefill -8 %, decode -6 %; a nanosleep of
// 20-400 ns between polls changes nothing.)
template <uint32_t HINT_NS = 0>
RK_DEVINL bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status, int code,
                         uint64_t limit_ns = 2000000000ull) {
  if (mbar_try_wait<HINT_NS>(bar, parity)) return true;
  const uint64_t t0 = global_timer_ns();
  for (uint32_t it = 1;; ++it) {
    if (mbar_try_wait<HINT_NS>(bar, parity)) return true;
    if ((it & 255u) == 0u) {
      if (*abort_flag || *reinterpret_cast<volatile int*>(status) != 0) { *abort_flag = 1; return false; }
      if (global_timer_ns() - t0 > limit_ns) break;
    }
  }
  *abort_flag = 1;
  atomicCAS(status, 0, code);
  return false;
}

// The same bound in a form that costs a dozen instructions where it is inlined: SM cycles instead of the global
// timer, and nothing recorded here.  The caller reports the failure (report_wait_failure) outside its hot loop.
constexpr long long kWaitLimitCycles = 4000000000ll;      // about two seconds at 1.9 GHz
RK_DEVINL bool mbar_wait_lean(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait<0>(bar, parity)) return true;
  const long long t0 = clock64();
  do {
    if (mbar_try_wait<0>(bar, parity)) return true;
  } while (!*abort_flag && clock64() - t0 < kWaitLimitCycles);
  return false;
}
RK_DEVINL void report_wait_failure(volatile int* abort_flag, int* status, int code) {
  *abort_flag = 1;
  atomicCAS(status, 0, code);
}

// Bounded wait for warps that are not on the critical path (producers, issuers, correction): between polls the
// warp sleeps `SLEEP_NS`, so that it leaves the issue slots of its scheduler to the warps that compute.  Same
// give-up rule as mbar_wait.
template <uint32_t SLEEP_NS>
RK_DEVINL bool mbar_wait_relaxed(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status, int code,
                                 uint64_t limit_ns = 2000000000ull) {
  if (mbar_try_wait<0>(bar, parity)) return true;
  const uint64_t t0 = global_timer_ns();
  for (uint32_t it = 1;; ++it) {
    __nanosleep(SLEEP_NS);
    if (mbar_try_wait<0>(bar, parity)) return true;
    if ((it & 63u) == 0u) {
      if (*abort_flag || *reinterpret_cast<volatile int*>(status) != 0) { *abort_flag = 1; return false; }
      if (global_timer_ns() - t0 > limit_ns) break;
    }
  }
  *abort_flag = 1;
  atomicCAS(status, 0, code);
  return false;
}

RK_DEVINL void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
RK_DEVINL void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// TMA: 3-D tiled load global -> shared, completion on an mbarrier.
RK_DEVINL void tma_load_3d(void* smem_dst, const void* tmap, uint64_t* bar, int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(tmap), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z) : "memory");
}
// TMA: 1-D bulk copy global -> shared (16-byte aligned, size multiple of 16).
RK_DEVINL void bulk_load_1d(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
RK_DEVINL void prefetch_tmap(const void* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}

// ---- TMEM / tcgen05 ----
RK_DEVINL void tmem_alloc(uint32_t* smem_dst, uint32_t ncols) {   // whole warp
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)), "r"(ncols) : "memory");
}
RK_DEVINL void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
RK_DEVINL void tmem_dealloc(uint32_t taddr, uint32_t ncols) {     // whole warp
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
RK_DEVINL void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
RK_DEVINL void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
RK_DEVINL void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
RK_DEVINL void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// mbarrier arrives once every tcgen05 op issued so far by this thread is done.
RK_DEVINL void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// Block-scaled MMA, operands in shared memory, E8M0 scales in TMEM:
// D[tmem] (+)= (A * sfa) . (B * sfb), one 32-deep K slice.
RK_DEVINL void mma_mxf8f6f4_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                               uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem) : "memory");
}
// 32 rows x 16 bytes of shared memory -> 4 TMEM columns, replicated into all
// four 32-lane quadrants (the scale-factor copy).
RK_DEVINL void tc_cp_32x128b_warpx4(uint32_t dst_tmem, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(dst_tmem), "l"(sdesc) : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns: thread i of the warp gets lane
// (base lane + i), registers r[0..31] = columns taddr.col + 0..31.
RK_DEVINL void tmem_ld32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
}
RK_DEVINL void tmem_ld16(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr) : "memory");
}
RK_DEVINL void tmem_st32(uint32_t taddr, const uint32_t* r) {
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

// Shared-memory matrix descriptor (sm_100 format): start address, leading and
// stride byte offsets in 16-byte units, descriptor version 1 at bits 46-47,
// layout type at bits 61-63 (0 = no swizzle, 2 = 128-byte swizzle).
RK_DEVINL uint64_t make_smem_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint32_t layout) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3FFFu);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)(layout & 7u) << 61;
  return d;
}
constexpr uint32_t kLayoutNone = 0, kLayoutSw128 = 2;

// Instruction descriptor of kind::mxf8f6f4.block_scale (dense):
//  [4,6) B scale id  [7,10) A format  [10,13) B format  [15] A MN-major  [16] B MN-major
//  [17,23) N>>3  [23] scale format (1 = E8M0)  [24,29) M>>4  [29,31) A scale id
// Hardware element-format ids: E4M3 0, E5M2 1, E2M3 3, E3M2 4, E2M1 5.
__host__ __device__ inline constexpr uint32_t hw_fmt_id(int fmt) { return fmt == 0 ? 0u : fmt == 1 ? 1u : fmt == 2 ? 3u : fmt == 3 ? 4u : 5u; }
__host__ __device__ inline constexpr uint32_t make_idesc(int a_fmt, int b_fmt, bool a_mn, bool b_mn, int M, int N) {
  return (hw_fmt_id(a_fmt) << 7) | (hw_fmt_id(b_fmt) << 10) | ((a_mn ? 1u : 0u) << 15) | ((b_mn ? 1u : 0u) << 16) |
         ((uint32_t)(N >> 3) << 17) | (1u << 23) | ((uint32_t)(M >> 4) << 24);
}
RK_DEVINL uint32_t idesc_with_sf(uint32_t idesc, uint32_t a_sf_id, uint32_t b_sf_id) {
  return idesc | (b_sf_id << 4) | (a_sf_id << 29);
}

RK_DEVINL float ex2_approx(float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
RK_DEVINL float rcp_approx(float x) { float y; asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }

}  // namespace rk
