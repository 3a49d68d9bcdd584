// Device-side activation functions and their derivatives for the fused linear layer.
//
// The set, the formulas and the conventions at the piecewise switch points follow
// attorch/act_kernels.py:14-628 of the reference (forward functions and *_grad functions;
// dispatch order in apply_act_func 631-732 and apply_act_func_grad 735-837).  Everything is
// evaluated in fp32.  Where the reference's literal formula overflows (logsigmoid, softplus,
// mish and mish' for |x| >~ 88) an algebraically equal, overflow-free form is used.
#pragma once
#include <cuda_runtime.h>

namespace ab200 {

// Activation ids shared with the host side (attorch_b200/acts.py keeps the same table).
enum Act : int {
  ACT_NONE = 0,
  ACT_SIGMOID = 1,
  ACT_LOGSIGMOID = 2,
  ACT_TANH = 3,
  ACT_RELU = 4,
  ACT_GELU = 5,
  ACT_GELUAPPROX = 6,
  ACT_SILU = 7,
  ACT_RELU6 = 8,
  ACT_HARDSIGMOID = 9,
  ACT_HARDTANH = 10,
  ACT_HARDSWISH = 11,
  ACT_SELU = 12,
  ACT_MISH = 13,
  ACT_SOFTPLUS = 14,
  ACT_SOFTSIGN = 15,
  ACT_TANHSHRINK = 16,
  ACT_LEAKY_RELU = 17,
  ACT_ELU = 18,
  ACT_CELU = 19,
  ACT_HARDSHRINK = 20,
  ACT_SOFTSHRINK = 21,
  ACT_COUNT = 22,
  // Backward only: the saved tensor already holds act'(Z) (written by a forward pass that was asked
  // to save the derivative), so dZ = dY * saved.
  ACT_SAVED_DERIVATIVE = 22,
  // Same, with the saved act'(Z) stored as fp16 whatever the type of dY and dZ (2-byte types only).
  ACT_SAVED_DERIVATIVE_F16 = 23
};

namespace actm {

// Single-instruction approximations (MUFU): 2^x and 1/x to about 2 ulp and 1 ulp.
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float rcp_approx(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float sigmoid(float x) {
  return rcp_approx(__fadd_rn(1.0f, ex2_approx(__fmul_rn(-1.44269504f, x))));
}
// tanh as 2*sigmoid(2x) - 1 (act_kernels.py:71-81).
__device__ __forceinline__ float tanh_(float x) { return 2.0f * sigmoid(2.0f * x) - 1.0f; }
// erf(x) by Abramowitz & Stegun 7.1.26: 1 - (a1 t + ... + a5 t^5) exp(-x^2), t = 1 / (1 + p |x|);
// absolute error below 1.5e-7 everywhere, i.e. at the resolution of fp32 near 1, for about a third
// of the instructions of the library erff.  The GEMM epilogue runs one warp per scheduler, so the
// instruction count of the activation is what decides whether it hides behind the main loop.
__device__ __forceinline__ float erf_fast(float x) {
  const float ax = fabsf(x);
  const float t = rcp_approx(fmaf(0.3275911f, ax, 1.0f));
  float poly = fmaf(1.061405429f, t, -1.453152027f);
  poly = fmaf(poly, t, 1.421413741f);
  poly = fmaf(poly, t, -0.284496736f);
  poly = fmaf(poly, t, 0.254829592f);
  const float r = 1.0f - poly * t * ex2_approx(-1.44269504f * ax * ax);
  return copysignf(r, x);
}
// log(1 + e^x) without overflow.
__device__ __forceinline__ float softplus(float x) {
  return fmaxf(x, 0.0f) + log1pf(__expf(-fabsf(x)));
}

constexpr float kSeluScale = 1.0507009873554805f;
constexpr float kSeluAlpha = 1.6732632423543772f;
constexpr float kRsqrt2 = 0.707106781f;
constexpr float kRsqrt2Pi = 0.39894228f;
constexpr float kSqrt2OverPi = 0.7978845608f;

template <int A>
__device__ __forceinline__ float fwd(float x, float p) {
  if constexpr (A == ACT_NONE) return x;
  if constexpr (A == ACT_SIGMOID) return sigmoid(x);
  if constexpr (A == ACT_LOGSIGMOID) return fminf(x, 0.0f) - log1pf(__expf(-fabsf(x)));
  if constexpr (A == ACT_TANH) return tanh_(x);
  if constexpr (A == ACT_RELU) return fmaxf(0.0f, x);
  if constexpr (A == ACT_GELU) return x * 0.5f * (1.0f + erf_fast(kRsqrt2 * x));
  if constexpr (A == ACT_GELUAPPROX)
    return x * 0.5f * (1.0f + tanh_(kSqrt2OverPi * x * (1.0f + 0.044715f * x * x)));
  if constexpr (A == ACT_SILU) return __fmul_rn(x, sigmoid(x));
  if constexpr (A == ACT_RELU6) return fminf(fmaxf(0.0f, x), 6.0f);
  if constexpr (A == ACT_HARDSIGMOID) return fmaxf(0.0f, fminf(1.0f, x / 6.0f + 0.5f));
  if constexpr (A == ACT_HARDTANH) return fmaxf(-1.0f, fminf(1.0f, x));
  if constexpr (A == ACT_HARDSWISH) return x * fminf(fmaxf(0.0f, x + 3.0f), 6.0f) / 6.0f;
  if constexpr (A == ACT_SELU)
    return kSeluScale * (fmaxf(0.0f, x) + fminf(0.0f, kSeluAlpha * (__expf(x) - 1.0f)));
  if constexpr (A == ACT_MISH) return x * tanh_(softplus(x));
  if constexpr (A == ACT_SOFTPLUS) return softplus(x);
  if constexpr (A == ACT_SOFTSIGN) return x / (1.0f + fabsf(x));
  if constexpr (A == ACT_TANHSHRINK) return x - tanh_(x);
  if constexpr (A == ACT_LEAKY_RELU) return fmaxf(0.0f, x) + p * fminf(0.0f, x);
  if constexpr (A == ACT_ELU) return x <= 0.0f ? p * (__expf(x) - 1.0f) : x;
  if constexpr (A == ACT_CELU)
    return fmaxf(0.0f, x) + fminf(0.0f, p * (__expf(__fdividef(x, p)) - 1.0f));
  if constexpr (A == ACT_HARDSHRINK) return fabsf(x) <= p ? 0.0f : x;
  if constexpr (A == ACT_SOFTSHRINK) return x > p ? x - p : (x < -p ? x + p : 0.0f);
  return x;
}

// d act(x) / dx.
template <int A>
__device__ __forceinline__ float grad(float x, float p) {
  if constexpr (A == ACT_NONE) return 1.0f;
  if constexpr (A == ACT_SIGMOID) {
    const float s = sigmoid(x);
    return s * (1.0f - s);
  }
  if constexpr (A == ACT_LOGSIGMOID) return sigmoid(-x);  // 1 / (1 + e^x)
  if constexpr (A == ACT_TANH) {
    const float t = tanh_(x);
    return 1.0f - t * t;
  }
  if constexpr (A == ACT_RELU) return x <= 0.0f ? 0.0f : 1.0f;
  if constexpr (A == ACT_GELU) {
    // Phi(x) + x * phi(x).  erf(x / sqrt 2) and phi(x) need the same exponential, exp(-x^2 / 2).
    const float e = ex2_approx(-0.72134752f * x * x);               // exp(-x^2 / 2)
    const float t = rcp_approx(fmaf(0.3275911f * kRsqrt2, fabsf(x), 1.0f));
    float poly = fmaf(1.061405429f, t, -1.453152027f);
    poly = fmaf(poly, t, 1.421413741f);
    poly = fmaf(poly, t, -0.284496736f);
    poly = fmaf(poly, t, 0.254829592f);
    const float half_erf = 0.5f - 0.5f * poly * t * e;        // erf(|x| / sqrt 2) / 2
    return fmaf(x * kRsqrt2Pi, e, 0.5f + copysignf(half_erf, x));
  }
  if constexpr (A == ACT_GELUAPPROX) {
    const float t = tanh_(kSqrt2OverPi * x * (1.0f + 0.044715f * x * x));
    return 0.5f * ((1.0f + t) +
                   x * (1.0f - t * t) * kSqrt2OverPi * (1.0f + 3.0f * 0.044715f * x * x));
  }
  if constexpr (A == ACT_SILU) {
    const float s = sigmoid(x);
    return __fmul_rn(s, __fmaf_rn(x, __fsub_rn(1.0f, s), 1.0f));     // spelled out: fwd_grad2 mirrors it
  }
  if constexpr (A == ACT_RELU6) return (x > 0.0f && x < 6.0f) ? 1.0f : 0.0f;
  if constexpr (A == ACT_HARDSIGMOID) return (x > -3.0f && x < 3.0f) ? (1.0f / 6.0f) : 0.0f;
  if constexpr (A == ACT_HARDTANH) return (x > -1.0f && x < 1.0f) ? 1.0f : 0.0f;
  if constexpr (A == ACT_HARDSWISH) return x < -3.0f ? 0.0f : (x <= 3.0f ? x / 3.0f + 0.5f : 1.0f);
  if constexpr (A == ACT_SELU) return kSeluScale * (x <= 0.0f ? kSeluAlpha * __expf(x) : 1.0f);
  if constexpr (A == ACT_MISH) {
    // tanh(sp) + x * sigmoid(x) * (1 - tanh(sp)^2), equal to the reference's rational form.
    const float t = tanh_(softplus(x));
    return t + x * sigmoid(x) * (1.0f - t * t);
  }
  if constexpr (A == ACT_SOFTPLUS) return sigmoid(x);
  if constexpr (A == ACT_SOFTSIGN) {
    const float d = 1.0f + fabsf(x);
    return 1.0f / (d * d);
  }
  if constexpr (A == ACT_TANHSHRINK) {
    const float t = tanh_(x);
    return t * t;  // 1 - (1 - tanh^2)
  }
  if constexpr (A == ACT_LEAKY_RELU) return x <= 0.0f ? p : 1.0f;
  if constexpr (A == ACT_ELU) return x <= 0.0f ? p * __expf(x) : 1.0f;
  if constexpr (A == ACT_CELU) return x <= 0.0f ? __expf(__fdividef(x, p)) : 1.0f;
  if constexpr (A == ACT_HARDSHRINK) return fabsf(x) <= p ? 0.0f : 1.0f;
  if constexpr (A == ACT_SOFTSHRINK) return fabsf(x) <= p ? 0.0f : 1.0f;
  return 1.0f;
}

// y = act(v) and g = act'(zr) in one go, for a forward pass that saves the derivative instead of the
// pre-activation.  zr is v rounded to the storage type, i.e. the pre-activation the reference would
// have stored and differentiated through (attorch/linear_layer.py:104-105, 143-146).  gelu, whose
// forward value and derivative need the same exponential, evaluates it once at v and carries the
// derivative over to zr with its own derivative, gelu''(v) = phi(v) (2 - v^2): the neglected term is
// of order (v - zr)^2, four orders of magnitude below the resolution g is stored with.
//
// The sequence of roundings is spelled out (no contraction left to the compiler) so that the two-element
// form below, which uses Blackwell's packed fp32 instructions, gives the same bits.
template <int A>
__device__ __forceinline__ void fwd_grad(float v, float zr, float p, float& y, float& g) {
  if constexpr (A == ACT_GELU) {
    const float vv = __fmul_rn(v, v);
    const float e = ex2_approx(__fmul_rn(vv, -0.72134752f));                             // exp(-v^2 / 2)
    const float t = rcp_approx(__fmaf_rn(0.3275911f * kRsqrt2, fabsf(v), 1.0f));
    float poly = __fmaf_rn(1.061405429f, t, -1.453152027f);
    poly = __fmaf_rn(poly, t, 1.421413741f);
    poly = __fmaf_rn(poly, t, -0.284496736f);
    poly = __fmaf_rn(poly, t, 0.254829592f);
    const float half_erf = __fmaf_rn(__fmul_rn(__fmul_rn(poly, t), e), -0.5f, 0.5f);    // erf(|v| / sqrt 2) / 2
    const float cdf = __fadd_rn(0.5f, copysignf(half_erf, v));
    const float pdf = __fmul_rn(e, kRsqrt2Pi);
    y = __fmul_rn(v, cdf);
    const float g1 = __fmaf_rn(v, pdf, cdf);
    const float q = __fmaf_rn(vv, -1.0f, 2.0f);                                          // 2 - v^2
    g = __fmaf_rn(__fmul_rn(pdf, q), __fmaf_rn(v, -1.0f, zr), g1);
  } else {
    y = fwd<A>(v, p);
    g = grad<A>(zr, p);
  }
}

// Packed fp32 arithmetic (sm_100: two IEEE round-to-nearest operations per instruction).
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
  float2 d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;"
      : "=l"(reinterpret_cast<unsigned long long&>(d))
      : "l"(reinterpret_cast<const unsigned long long&>(a)), "l"(reinterpret_cast<const unsigned long long&>(b)),
        "l"(reinterpret_cast<const unsigned long long&>(c)));
  return d;
}
__device__ __forceinline__ float2 mul2(float2 a, float2 b) {
  float2 d;
  asm("mul.rn.f32x2 %0, %1, %2;"
      : "=l"(reinterpret_cast<unsigned long long&>(d))
      : "l"(reinterpret_cast<const unsigned long long&>(a)), "l"(reinterpret_cast<const unsigned long long&>(b)));
  return d;
}
__device__ __forceinline__ float2 add2(float2 a, float2 b) {
  float2 d;
  asm("add.rn.f32x2 %0, %1, %2;"
      : "=l"(reinterpret_cast<unsigned long long&>(d))
      : "l"(reinterpret_cast<const unsigned long long&>(a)), "l"(reinterpret_cast<const unsigned long long&>(b)));
  return d;
}
__device__ __forceinline__ float2 both(float c) { return make_float2(c, c); }

// fwd_grad for two elements at once; for gelu the polynomial, the products and the sums run as packed
// instructions (the two exponentials and reciprocals stay scalar).  Same bits as two calls of fwd_grad.
template <int A>
__device__ __forceinline__ void fwd_grad2(float v0, float v1, float zr0, float zr1, float p, float& y0, float& y1,
                                          float& g0, float& g1) {
  if constexpr (A == ACT_GELU) {
    const float2 v = make_float2(v0, v1);
    const float2 vv = mul2(v, v);
    const float2 ea = mul2(vv, both(-0.72134752f));
    const float2 e = make_float2(ex2_approx(ea.x), ex2_approx(ea.y));
    // Scalar: the absolute value is an operand modifier of the scalar instruction, not an instruction.
    const float2 t = make_float2(rcp_approx(__fmaf_rn(0.3275911f * kRsqrt2, fabsf(v0), 1.0f)),
                                 rcp_approx(__fmaf_rn(0.3275911f * kRsqrt2, fabsf(v1), 1.0f)));
    float2 poly = fma2(both(1.061405429f), t, both(-1.453152027f));
    poly = fma2(poly, t, both(1.421413741f));
    poly = fma2(poly, t, both(-0.284496736f));
    poly = fma2(poly, t, both(0.254829592f));
    const float2 half_erf = fma2(mul2(mul2(poly, t), e), both(-0.5f), both(0.5f));
    const float2 cdf = add2(both(0.5f), make_float2(copysignf(half_erf.x, v0), copysignf(half_erf.y, v1)));
    const float2 pdf = mul2(e, both(kRsqrt2Pi));
    const float2 y = mul2(v, cdf);
    const float2 ga = fma2(v, pdf, cdf);
    const float2 q = fma2(vv, both(-1.0f), both(2.0f));
    const float2 g = fma2(mul2(pdf, q), fma2(v, both(-1.0f), make_float2(zr0, zr1)), ga);
    y0 = y.x; y1 = y.y; g0 = g.x; g1 = g.y;
  } else if constexpr (A == ACT_SILU) {
    // y = v sigmoid(v), g = s (zr (1 - s) + 1) with s = sigmoid(zr): four sigmoids, two packed pairs.
    const float2 v = make_float2(v0, v1), zr = make_float2(zr0, zr1);
    const float2 ev = mul2(both(-1.44269504f), v), ez = mul2(both(-1.44269504f), zr);
    const float2 dv = add2(both(1.0f), make_float2(ex2_approx(ev.x), ex2_approx(ev.y)));
    const float2 dz = add2(both(1.0f), make_float2(ex2_approx(ez.x), ex2_approx(ez.y)));
    const float2 sv = make_float2(rcp_approx(dv.x), rcp_approx(dv.y));
    const float2 sz = make_float2(rcp_approx(dz.x), rcp_approx(dz.y));
    const float2 y = mul2(v, sv);
    const float2 g = mul2(sz, fma2(zr, fma2(sz, both(-1.0f), both(1.0f)), both(1.0f)));
    y0 = y.x; y1 = y.y; g0 = g.x; g1 = g.y;
  } else {
    fwd_grad<A>(v0, zr0, p, y0, g0);
    fwd_grad<A>(v1, zr1, p, y1, g1);
  }
}

}  // namespace actm

// Calls f.template operator()<A>() with the runtime id turned into a compile-time constant,
// so that loops over elements sit inside the switch and not the other way round.
template <class F>
__device__ __forceinline__ void dispatch_act(int act, F&& f) {
  switch (act) {
#define AB200_CASE(A) \
  case A:             \
    f.template operator()<A>(); \
    break;
    AB200_CASE(ACT_SIGMOID)
    AB200_CASE(ACT_LOGSIGMOID)
    AB200_CASE(ACT_TANH)
    AB200_CASE(ACT_RELU)
    AB200_CASE(ACT_GELU)
    AB200_CASE(ACT_GELUAPPROX)
    AB200_CASE(ACT_SILU)
    AB200_CASE(ACT_RELU6)
    AB200_CASE(ACT_HARDSIGMOID)
    AB200_CASE(ACT_HARDTANH)
    AB200_CASE(ACT_HARDSWISH)
    AB200_CASE(ACT_SELU)
    AB200_CASE(ACT_MISH)
    AB200_CASE(ACT_SOFTPLUS)
    AB200_CASE(ACT_SOFTSIGN)
    AB200_CASE(ACT_TANHSHRINK)
    AB200_CASE(ACT_LEAKY_RELU)
    AB200_CASE(ACT_ELU)
    AB200_CASE(ACT_CELU)
    AB200_CASE(ACT_HARDSHRINK)
    AB200_CASE(ACT_SOFTSHRINK)
#undef AB200_CASE
    default:
      f.template operator()<ACT_NONE>();
      break;
  }
}

// In-place activation of n consecutive fp32 values.
template <int N>
__device__ __forceinline__ void act_fwd_inplace(float (&v)[N], int act, float p) {
  if (act == ACT_NONE) return;
  dispatch_act(act, [&]<int A>() {
#pragma unroll
    for (int i = 0; i < N; ++i) v[i] = actm::fwd<A>(v[i], p);
  });
}

// v[i] <- act(v[i]) and g[i] <- act'(.), see actm::fwd_grad; zr[i] is v[i] rounded to storage.
template <int N>
__device__ __forceinline__ void act_fwd_grad(float (&v)[N], const float (&zr)[N], float (&g)[N], int act, float p) {
  dispatch_act(act, [&]<int A>() {
#pragma unroll
    for (int i = 0; i + 1 < N; i += 2) {
      float y0, y1;
      actm::fwd_grad2<A>(v[i], v[i + 1], zr[i], zr[i + 1], p, y0, y1, g[i], g[i + 1]);
      v[i] = y0;
      v[i + 1] = y1;
    }
    if constexpr (N % 2 == 1) {
      float y;
      actm::fwd_grad<A>(v[N - 1], zr[N - 1], p, y, g[N - 1]);
      v[N - 1] = y;
    }
  });
}

// g[i] *= act'(z[i]).
template <int N>
__device__ __forceinline__ void act_grad_mul(float (&g)[N], const float (&z)[N], int act, float p) {
  if (act == ACT_NONE) return;
  if (act == ACT_SAVED_DERIVATIVE || act == ACT_SAVED_DERIVATIVE_F16) {
#pragma unroll
    for (int i = 0; i < N; ++i) g[i] *= z[i];
    return;
  }
  dispatch_act(act, [&]<int A>() {
#pragma unroll
    for (int i = 0; i < N; ++i) g[i] *= actm::grad<A>(z[i], p);
  });
}

}  // namespace ab200
