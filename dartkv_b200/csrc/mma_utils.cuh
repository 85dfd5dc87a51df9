// PTX wrappers used by the tensor-core decode kernel: bulk async copies with mbarrier completion,
// packed 16-bit arithmetic with round-to-nearest-even, and warp-level m16n8k16 MMA.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include "../../include/dartkv_b200.h"

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// ---------------------------------------------------------------------------- mbarrier + bulk copy
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Bounded wait: returns false if the phase did not complete within the spin budget.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  const uint32_t addr = smem_u32(bar);
  for (int spin = 0; spin < (1 << 22); ++spin) {
    uint32_t done;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(done)
        : "r"(addr), "r"(parity)
        : "memory");
    if (done) return true;
  }
  return false;
}
// 1-D bulk copy global -> shared of `bytes` (multiple of 16, both addresses 16-byte aligned);
// completion is signalled on `bar` as transaction bytes.  No multicast.
__device__ __forceinline__ void bulk_copy_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(dst)),
               "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

// ---------------------------------------------------------------------------- packed 16-bit math
template <int DT> struct Half2Ops;

template <> struct Half2Ops<DARTKV_BF16> {
  static __device__ __forceinline__ uint32_t fma(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
  }
  static __device__ __forceinline__ uint32_t add(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("add.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
  }
  static __device__ __forceinline__ uint32_t mul(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
  }
  static __device__ __forceinline__ uint16_t from_float(float x) { return __bfloat16_as_ushort(__float2bfloat16_rn(x)); }
  static __device__ __forceinline__ float to_float(uint16_t x) { return __bfloat162float(__ushort_as_bfloat16(x)); }
  static __device__ __forceinline__ void mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  }
  // code positions (2-bit field index inside a 16-bit half) that sit in the mantissa with unit weight
  // when OR-ed into the magic exponent: 128 + c, 32 + c, 8 + c
  static __host__ __device__ constexpr uint32_t magic(int j) { return j == 0 ? 0x43004300u : (j == 1 ? 0x42004200u : 0x41004100u); }
  static __host__ __device__ constexpr uint32_t neg_magic(int j) { return magic(j) | 0x80008000u; }
  static constexpr int kFirstPos = 0;
};

template <> struct Half2Ops<DARTKV_F16> {
  static __device__ __forceinline__ uint32_t fma(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
  }
  static __device__ __forceinline__ uint32_t add(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("add.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
  }
  static __device__ __forceinline__ uint32_t mul(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
  }
  static __device__ __forceinline__ uint16_t from_float(float x) { return __half_as_ushort(__float2half_rn(x)); }
  static __device__ __forceinline__ float to_float(uint16_t x) { return __half2float(__ushort_as_half(x)); }
  static __device__ __forceinline__ void mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  }
  // positions 2,3,4 (bits 4..9 of the mantissa): 64 + c, 16 + c, 4 + c keep -magic*scale far from overflow
  static __host__ __device__ constexpr uint32_t magic(int j) { return j == 0 ? 0x54005400u : (j == 1 ? 0x4C004C00u : 0x44004400u); }
  static __host__ __device__ constexpr uint32_t neg_magic(int j) { return magic(j) | 0x80008000u; }
  static constexpr int kFirstPos = 2;
};

// two floats -> one register of two 16-bit numbers (round to nearest even), `lo` in the low half
template <int DT> __device__ __forceinline__ uint32_t pack16(float lo, float hi) {
  uint32_t d;
  if (DT == DARTKV_F16) asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
  else asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
  return d;
}
// the two 16-bit numbers of a register as floats
template <int DT> __device__ __forceinline__ void unpack16(uint32_t x, float& lo, float& hi) {
  if (DT == DARTKV_F16) {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&x));
    lo = f.x; hi = f.y;
  } else {
    lo = __uint_as_float(x << 16); hi = __uint_as_float(x & 0xFFFF0000u);
  }
}

// one register of two 16-bit numbers of dtype FROM as dtype TO (round to nearest even; the cast of the dequantized
// value from the metadata dtype to the cache dtype when the two differ)
template <int FROM, int TO> __device__ __forceinline__ uint32_t cast16(uint32_t x) {
  if (FROM == TO) return x;
  float lo, hi;
  unpack16<FROM>(x, lo, hi);
  return pack16<TO>(lo, hi);
}

// (a & b) | c in one LOP3; b and c are kept in registers (a logic op takes at most one immediate)
__device__ __forceinline__ uint32_t and_or(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
// a value the compiler must keep in a register instead of re-materializing as an immediate
__device__ __forceinline__ uint32_t reg_const(uint32_t v) {
  uint32_t r;
  asm volatile("mov.b32 %0, %1;" : "=r"(r) : "r"(v));
  return r;
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// masks and magic exponents of the three in-mantissa code positions, held in registers
template <int DT>
struct CodeConsts {
  uint32_t mask[3], magic[3];
  __device__ __forceinline__ void init() {
    using H = Half2Ops<DT>;
#pragma unroll
    for (int j = 0; j < 3; ++j) {
      mask[j] = reg_const(0x00030003u << (2 * (H::kFirstPos + j)));
      magic[j] = reg_const(H::magic(j));
    }
  }
};

// shift a packed-code word so that code index `code` of each 16-bit half lands at field position `pos`
__device__ __forceinline__ uint32_t align_codes(uint32_t w, int code, int pos, int extra_left = 0) {
  const int left = 2 * pos + extra_left - 2 * code;
  return left >= 0 ? (w << left) : (w >> (-left));
}

// timing experiments only (a library built with these computes garbage): drop one of the two packed ops
#if defined(PEROP_SKIP_ADD)
#define DQ_ADD(t, z) (t)
#else
#define DQ_ADD(t, z) H::add((t), (z))
#endif
#if defined(PEROP_SKIP_FMA)
#define DQ_FMA(m, s, ms) (m)
#else
#define DQ_FMA(m, s, ms) H::fma((m), (s), (ms))
#endif

// ---------------------------------------------------------------------------- exact packed dequantization
// A packed word holds sixteen 2-bit codes; code u of the low half and code u of the high half share
// a (scale, zero) pair, so one 32-bit register of two 16-bit floats is produced per u:
//   m = magic + code          (code bits OR-ed into the mantissa, exact)
//   t = fma(m, s, -magic*s)   = round16(code * s)
//   r = add(t, z)             = round16(round16(code * s) + z)
// which is the reference's per-op rounding in the metadata dtype (src/dart/quantization.py:103-106).
template <int DT>
__device__ __forceinline__ void dequant_word2(const CodeConsts<DT>& k, uint32_t w, uint32_t ss, uint32_t zz,
                                              uint32_t ms0, uint32_t ms1, uint32_t ms2, uint32_t (&r)[8]) {
  using H = Half2Ops<DT>;
  constexpr int P0 = H::kFirstPos;
#pragma unroll
  for (int grp = 0; grp < 3; ++grp) {
    const uint32_t x = align_codes(w, 3 * grp, P0);
#pragma unroll
    for (int j = 0; j < 3; ++j) {
      const int u = 3 * grp + j;
      if (u < 8) {
        const uint32_t m = and_or(x, k.mask[j], k.magic[j]);
        const uint32_t ms = j == 0 ? ms0 : (j == 1 ? ms1 : ms2);
        r[u] = DQ_ADD(DQ_FMA(m, ss, ms), zz);
      }
    }
  }
}

// 4-bit codes split over a low-bit word and a high-bit word (promoted key channels): code = low | high << 2
template <int DT>
__device__ __forceinline__ void dequant_word4(const CodeConsts<DT>& k, uint32_t wl, uint32_t wh, uint32_t ss,
                                              uint32_t zz, uint32_t ms0, uint32_t ms1, uint32_t (&r)[8]) {
  using H = Half2Ops<DT>;
  constexpr int P0 = H::kFirstPos;
#pragma unroll
  for (int grp = 0; grp < 4; ++grp) {
    const uint32_t xl = align_codes(wl, 2 * grp, P0);
    const uint32_t xh = align_codes(wh, 2 * grp, P0, 2);
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int u = 2 * grp + j;
      // the high field of position j sits where the low field of position j+1 does
      const uint32_t m = and_or(xh, k.mask[j + 1], and_or(xl, k.mask[j], k.magic[j]));
      r[u] = DQ_ADD(DQ_FMA(m, ss, j == 0 ? ms0 : ms1), zz);
    }
  }
}

// ---------------------------------------------------------------------------- half-word variants
// Two warps share a staged page; warp half HF owns codes 4*HF .. 4*HF+3 of every 16-bit half.
template <int DT, int HF>
__device__ __forceinline__ void dequant_half2(const CodeConsts<DT>& k, uint32_t w, uint32_t ss, uint32_t zz,
                                              uint32_t ms0, uint32_t ms1, uint32_t ms2, uint32_t (&r)[4]) {
  using H = Half2Ops<DT>;
  constexpr int P0 = H::kFirstPos;
  if (HF == 0) {
    const uint32_t xa = align_codes(w, 0, P0);   // codes 0,1,2 at positions 0,1,2
    const uint32_t xb = align_codes(w, 3, P0);   // code 3 at position 0
    r[0] = DQ_ADD(DQ_FMA(and_or(xa, k.mask[0], k.magic[0]), ss, ms0), zz);
    r[1] = DQ_ADD(DQ_FMA(and_or(xa, k.mask[1], k.magic[1]), ss, ms1), zz);
    r[2] = DQ_ADD(DQ_FMA(and_or(xa, k.mask[2], k.magic[2]), ss, ms2), zz);
    r[3] = DQ_ADD(DQ_FMA(and_or(xb, k.mask[0], k.magic[0]), ss, ms0), zz);
  } else {
    const uint32_t xa = align_codes(w, 3, P0);   // codes 4,5 at positions 1,2
    const uint32_t xb = align_codes(w, 6, P0);   // codes 6,7 at positions 0,1
    r[0] = DQ_ADD(DQ_FMA(and_or(xa, k.mask[1], k.magic[1]), ss, ms1), zz);
    r[1] = DQ_ADD(DQ_FMA(and_or(xa, k.mask[2], k.magic[2]), ss, ms2), zz);
    r[2] = DQ_ADD(DQ_FMA(and_or(xb, k.mask[0], k.magic[0]), ss, ms0), zz);
    r[3] = DQ_ADD(DQ_FMA(and_or(xb, k.mask[1], k.magic[1]), ss, ms1), zz);
  }
}

template <int DT, int HF>
__device__ __forceinline__ void dequant_half4(const CodeConsts<DT>& k, uint32_t wl, uint32_t wh, uint32_t ss,
                                              uint32_t zz, uint32_t ms0, uint32_t ms1, uint32_t (&r)[4]) {
  using H = Half2Ops<DT>;
  constexpr int P0 = H::kFirstPos;
#pragma unroll
  for (int grp = 0; grp < 2; ++grp) {
    const int code = 4 * HF + 2 * grp;
    const uint32_t xl = align_codes(wl, code, P0);
    const uint32_t xh = align_codes(wh, code, P0, 2);
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const uint32_t m = and_or(xh, k.mask[j + 1], and_or(xl, k.mask[j], k.magic[j]));
      r[2 * grp + j] = DQ_ADD(DQ_FMA(m, ss, j == 0 ? ms0 : ms1), zz);
    }
  }
}
