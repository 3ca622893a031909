// Per-element optimizer arithmetic shared by the fused wgrad epilogue and the optimizer-only
// kernels, following the reference's update (src/fused_grad_optimizer/kernel.py:300-317 AdamW,
// :203-205 SGD, :424-478 int8 moments, src/fused_grad_optimizer/kernel_fp8_state.py:272-295 fp8
// moments).
//
// What is reproduced bit for bit (given the same fp32 gradient) by a CPU restatement compiled
// without contraction: the new moments m', v' (explicitly rounded multiplies and adds in the
// reference's order), the int8 / fp8 codes and their scales (correctly rounded quotients), and the
// SGD / momentum / Lion weights (multiplies and adds only).
// What is NOT bit-reproduced: the AdamW weight.  Its bias-corrected quotient lr*m_hat/(sqrt(v_hat)
// + eps) is evaluated with the hardware's approximate reciprocal and square root and folded
// constants (relative error ~1e-6 of an update that is itself ~1e-3 of W), which keeps the stored
// weight within one bf16 ULP of the IEEE evaluation and removes three IEEE divisions and a square
// root from every element of an epilogue that otherwise could not keep up with HBM.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <stdint.h>

namespace forge {

enum Optimizer : int { OPT_ADAMW = 0, OPT_SGD = 1, OPT_SGDM = 2, OPT_LION = 3 };

// storage of the optimizer moments
enum StateMode : int {
  ST_NONE = 0,        // no moments (plain SGD)
  ST_F32 = 1,         // fp32 moments
  ST_BF16 = 2,        // bf16 moments
  ST_INT8 = 3,        // int8 codes + one fp32 absmax scale per (row, 64 columns)
  ST_FP8_BLOCK = 4,   // e4m3 codes for m and v + one fp32 absmax scale per (row, 64 columns)
  ST_FP8_TENSOR = 5   // e4m3 m / e5m2 v + one fp32 scale per tensor (delayed scaling)
};

enum DType : int { DT_BF16 = 0, DT_F32 = 1 };

// hyper-parameters, narrowed to fp32 on the host exactly as the reference's kernel arguments are
struct Hyper {
  float lr;
  float beta1;
  float beta2;
  float eps;
  float weight_decay;
  float bc1;             // 1 - beta1^step, evaluated in double on the host then narrowed
  float bc2;             // 1 - beta2^step
  float one_m_beta1;     // fp32(1 - beta1), the difference taken in double
  float one_m_beta2;
  float decay;           // fp32(1 - lr * weight_decay), evaluated in double
  float momentum;        // SGD momentum
  int nesterov;
  float lr_over_bc1;     // fp32(lr / bc1), quotient taken in double
  float inv_bc2;         // fp32(1 / bc2)
};

__device__ __forceinline__ float f_mul(float a, float b) { return __fmul_rn(a, b); }
__device__ __forceinline__ float f_add(float a, float b) { return __fadd_rn(a, b); }
__device__ __forceinline__ float f_sub(float a, float b) { return __fsub_rn(a, b); }
__device__ __forceinline__ float f_div(float a, float b) { return __fdiv_rn(a, b); }
__device__ __forceinline__ float f_sqrt(float a) { return __fsqrt_rn(a); }

__device__ __forceinline__ float sqrt_approx(float x) {
  float y;
  asm("sqrt.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float rcp_approx(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Correctly rounded a / b given rb = RN(1 / b): one multiply and two fused corrections (Markstein).
// Valid while no intermediate underflows, which holds for the quantiser's operands.
__device__ __forceinline__ float div_by_rcp(float a, float b, float rb) {
  const float q = __fmul_rn(a, rb);
  const float r = __fmaf_rn(-q, b, a);
  return __fmaf_rn(r, rb, q);
}

// AdamW: returns w', updates m and v in place (unrounded fp32 values, bit-reproducible)
__device__ __forceinline__ float adamw_update(float w, float g, float& m, float& v, const Hyper& h) {
  m = f_add(f_mul(h.beta1, m), f_mul(h.one_m_beta1, g));
  v = f_add(f_mul(h.beta2, v), f_mul(f_mul(h.one_m_beta2, g), g));
  const float den = sqrt_approx(v * h.inv_bc2) + h.eps;
  const float q = (m * h.lr_over_bc1) * rcp_approx(den);
  return __fmaf_rn(w, h.decay, -q);
}

// Packed fp32 arithmetic of sm_100 on register pairs.  Written as PTX with the rounding mode spelled
// out: an add or mul that names its rounding is never contracted into an fma, and every lane rounds
// exactly like the scalar instruction.
__device__ __forceinline__ float2 fmul2(float2 a, float2 b) {
  float2 d;
  asm("{\n\t.reg .b64 ra, rb, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t"
      "mul.rn.f32x2 rd, ra, rb;\n\tmov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d.x), "=f"(d.y)
      : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
  return d;
}
__device__ __forceinline__ float2 fadd2(float2 a, float2 b) {
  float2 d;
  asm("{\n\t.reg .b64 ra, rb, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t"
      "add.rn.f32x2 rd, ra, rb;\n\tmov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d.x), "=f"(d.y)
      : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
  return d;
}
__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) {
  float2 d;
  asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\tmov.b64 rc, {%6, %7};\n\t"
      "fma.rn.f32x2 rd, ra, rb, rc;\n\tmov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d.x), "=f"(d.y)
      : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y), "f"(c.x), "f"(c.y));
  return d;
}

// The same update on two neighbouring elements with the packed fp32 instructions of sm_100
// (each lane rounds exactly like the scalar form, so the results are
// bit-identical to adamw_update); halves the instruction count of everything but the two
// special-function evaluations.
__device__ __forceinline__ float2 adamw_update2(float2 w, float2 g, float2& m, float2& v, const Hyper& h) {
  const float2 b1 = make_float2(h.beta1, h.beta1), c1 = make_float2(h.one_m_beta1, h.one_m_beta1);
  const float2 b2 = make_float2(h.beta2, h.beta2), c2 = make_float2(h.one_m_beta2, h.one_m_beta2);
  // The products are packed; the sums are scalar adds.  A packed add fed by a packed multiply came
  // out of the assembler as one fused operation (m', v' off by an ulp in 5 % of the elements), and so
  // did a packed multiply-add with the multiplier one standing in for the add; the moments must
  // match the separately rounded reference arithmetic bit for bit.
  const float2 pm = fmul2(b1, m), pg = fmul2(c1, g);
  m = make_float2(f_add(pm.x, pg.x), f_add(pm.y, pg.y));
  const float2 pv = fmul2(b2, v), pgg = fmul2(fmul2(c2, g), g);
  v = make_float2(f_add(pv.x, pgg.x), f_add(pv.y, pgg.y));
  const float2 vh = fmul2(v, make_float2(h.inv_bc2, h.inv_bc2));
  const float2 den = fadd2(make_float2(sqrt_approx(vh.x), sqrt_approx(vh.y)), make_float2(h.eps, h.eps));
  const float2 mh = fmul2(m, make_float2(-h.lr_over_bc1, -h.lr_over_bc1));
  const float2 nq = fmul2(mh, make_float2(rcp_approx(den.x), rcp_approx(den.y)));
  return ffma2(w, make_float2(h.decay, h.decay), nq);
}

// SGD with decoupled decay: w' = w (1 - lr wd) - lr g
__device__ __forceinline__ float sgd_update(float w, float g, const Hyper& h) {
  return f_sub(f_mul(w, h.decay), f_mul(h.lr, g));
}

// SGD with momentum (buffer semantics of torch.optim.SGD with dampening 0; a zero-initialised
// buffer gives buf = g on the first step) and the reference's decoupled decay.
__device__ __forceinline__ float sgdm_update(float w, float g, float& buf, const Hyper& h) {
  buf = f_add(f_mul(h.momentum, buf), g);
  const float u = h.nesterov ? f_add(g, f_mul(h.momentum, buf)) : buf;
  return f_sub(f_mul(w, h.decay), f_mul(h.lr, u));
}

// Lion: u = sign(beta1 m + (1-beta1) g); w' = w (1 - lr wd) - lr u; m' = beta2 m + (1-beta2) g
__device__ __forceinline__ float lion_update(float w, float g, float& m, const Hyper& h) {
  const float c = f_add(f_mul(h.beta1, m), f_mul(h.one_m_beta1, g));
  const float u = (c > 0.0f) ? 1.0f : ((c < 0.0f) ? -1.0f : 0.0f);
  m = f_add(f_mul(h.beta2, m), f_mul(h.one_m_beta2, g));
  return f_sub(f_mul(w, h.decay), f_mul(h.lr, u));
}

// ----- quantisers -----------------------------------------------------------------------------
// int8: scale = absmax / 127 + 1e-12 ; code = clamp(rint(x / scale), -127, 127)
// Correctly rounded a / C for a compile-time constant C: Markstein's correction with rb = RN(1 / C)
// (three instructions instead of the ~30 of an IEEE division); operands so small that an
// intermediate could be subnormal take the division.
template <int C>
__device__ __forceinline__ float div_by_const(float a) {
  constexpr float b = static_cast<float>(C);
  constexpr float rb = 1.0f / b;
  if (a < 1e-30f) return f_div(a, b);
  return div_by_rcp(a, b, rb);
}
// correctly rounded 1 / x (identical to f_div(1, x), a third of the instructions)
__device__ __forceinline__ float f_rcp(float x) { return __frcp_rn(x); }

__device__ __forceinline__ float int8_scale(float absmax) {
  return f_add(div_by_const<127>(absmax), 1e-12f);
}
// `rscale` = RN(1 / scale), computed once per block with the IEEE reciprocal
__device__ __forceinline__ int int8_code(float x, float scale, float rscale) {
  const float q = rintf(div_by_rcp(x, scale, rscale));
  return static_cast<int>(fminf(fmaxf(q, -127.0f), 127.0f));
}
// Same code in one instruction: round-to-nearest-even conversion with saturation.  The saturation
// bound of the instruction is [-128, 127]; -128 cannot occur because scale > absmax / 127 keeps
// |x / scale| < 127.5, so the result equals clamp(rint(x / scale), -127, 127).
__device__ __forceinline__ uint32_t int8_code_bits(float x, float scale, float rscale) {
  int32_t q;
  asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(q) : "f"(div_by_rcp(x, scale, rscale)));
  return static_cast<uint32_t>(q) & 0xFFu;
}
// max(a, b, c) in one instruction (three-input form of sm_100)
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

// ---- the same quantiser arithmetic on element pairs, without the conversion unit ----------------
// Correctly rounded a / b on two elements given neg_b = -b and rb = RN(1 / b) (div_by_rcp, packed).
__device__ __forceinline__ float2 div2_by_rcp(float2 a, float2 neg_b, float2 rb) {
  const float2 q = fmul2(a, rb);
  const float2 r = ffma2(q, neg_b, a);
  return ffma2(r, rb, q);
}
// Two int8 codes -> fp32, exactly.  `biased` holds four codes with their sign bits flipped
// (code + 128 as an unsigned byte); a byte dropped into the mantissa of 2^23 reads as 2^23 + byte,
// and subtracting 2^23 + 128 leaves the code.  `first` is 0 or 2 (which pair of the word).
__device__ __forceinline__ float2 int8x2_to_float(uint32_t biased, int first) {
  const float f0 = __uint_as_float(__byte_perm(biased, 0x4B000000u, 0x7540u + first));
  const float f1 = __uint_as_float(__byte_perm(biased, 0x4B000000u, 0x7541u + first));
  return fadd2(make_float2(f0, f1), make_float2(-8388736.0f, -8388736.0f));
}
// Two NON-NEGATIVE int8 codes (second moments: 0..127) -> fp32, exactly; no sign-bit flip needed: the
// byte itself dropped into the mantissa of 2^23 reads as 2^23 + code.
__device__ __forceinline__ float2 uint8x2_to_float(uint32_t codes, int first) {
  const float f0 = __uint_as_float(__byte_perm(codes, 0x4B000000u, 0x7540u + first));
  const float f1 = __uint_as_float(__byte_perm(codes, 0x4B000000u, 0x7541u + first));
  return fadd2(make_float2(f0, f1), make_float2(-8388608.0f, -8388608.0f));
}
// rint() of two quotients as the low bytes of q + 1.5 * 2^23 (round to nearest even; two's
// complement in the mantissa).  |q| < 127.5 by construction of the scale, so no clamp is needed.
// Returns the two sums; int8x4_pack gathers their low bytes.
__device__ __forceinline__ float2 int8x2_round(float2 q) {
  return fadd2(q, make_float2(12582912.0f, 12582912.0f));
}
__device__ __forceinline__ uint32_t int8x4_pack(float2 r01, float2 r23) {
  const uint32_t lo = __byte_perm(__float_as_uint(r01.x), __float_as_uint(r01.y), 0x0040u);
  const uint32_t hi = __byte_perm(__float_as_uint(r23.x), __float_as_uint(r23.y), 0x0040u);
  return __byte_perm(lo, hi, 0x5410u);
}

// two e4m3 codes at once (round to nearest even, saturate to +-448): low byte = lo, next byte = hi
__device__ __forceinline__ uint32_t e4m3x2_code_bits(float lo, float hi) {
  uint16_t r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
  return static_cast<uint32_t>(r);
}
// two e4m3 codes -> two floats
__device__ __forceinline__ void e4m3x2_to_float(uint32_t two_codes, float& lo, float& hi) {
  uint32_t h2;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"(static_cast<uint16_t>(two_codes)));
  const __half2 hh = *reinterpret_cast<const __half2*>(&h2);
  lo = __low2float(hh);
  hi = __high2float(hh);
}
__device__ __forceinline__ uint32_t e5m2x2_code_bits(float lo, float hi) {
  uint16_t r;
  asm("cvt.rn.satfinite.e5m2x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
  return static_cast<uint32_t>(r);
}
__device__ __forceinline__ void e5m2x2_to_float(uint32_t two_codes, float& lo, float& hi) {
  uint32_t h2;
  asm("cvt.rn.f16x2.e5m2x2 %0, %1;" : "=r"(h2) : "h"(static_cast<uint16_t>(two_codes)));
  const __half2 hh = *reinterpret_cast<const __half2*>(&h2);
  lo = __low2float(hh);
  hi = __high2float(hh);
}
// e4m3 per-block: scale = absmax / 448 + 1e-12 ; code = e4m3_rne(clamp(x / scale, +-448))
__device__ __forceinline__ float fp8blk_scale(float absmax) {
  return f_add(div_by_const<448>(absmax), 1e-12f);
}
__device__ __forceinline__ uint8_t e4m3_code(float x_scaled) {
  const float c = fminf(fmaxf(x_scaled, -448.0f), 448.0f);
  return static_cast<uint8_t>(__nv_cvt_float_to_fp8(c, __NV_SATFINITE, __NV_E4M3));
}
__device__ __forceinline__ uint8_t e5m2_code(float x_scaled) {
  const float c = fminf(fmaxf(x_scaled, -57344.0f), 57344.0f);
  return static_cast<uint8_t>(__nv_cvt_float_to_fp8(c, __NV_SATFINITE, __NV_E5M2));
}
__device__ __forceinline__ float e4m3_to_float(uint8_t c) {
  const __half_raw hr = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(c), __NV_E4M3);
  return __half2float(__half(hr));
}
__device__ __forceinline__ float e5m2_to_float(uint8_t c) {
  const __half_raw hr = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(c), __NV_E5M2);
  return __half2float(__half(hr));
}

__device__ __forceinline__ float bf16_bits_to_float(uint32_t b16) {
  return __uint_as_float(b16 << 16);
}
__device__ __forceinline__ uint32_t float_to_bf16_bits(float f) {
  return static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(f)));
}

}  // namespace forge
