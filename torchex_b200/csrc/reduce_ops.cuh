// Reduce operators shared by the segment-reduction kernels: the running state of
// one lane (VEC channels), how a feature row is added to it, how two partial
// states of the same segment are merged, and how a state is packed into 32-bit
// words for shared memory, the workspace or a warp shuffle.
#pragma once

#include <cfloat>
#include <cstdint>

#include "common.cuh"

#ifndef TEXB_PACKED_F32X2
#define TEXB_PACKED_F32X2 1
#endif

namespace texb {

// ---- operators --------------------------------------------------------------
// State<VEC> lives in registers; pack / unpack move it through two arrays of
// VEC 32-bit words (shared memory or the workspace).

struct OpSumComp {  // fp32 sum + error-free two-sum: (s, c) with s + c the exact running sum
  static constexpr bool kRawBf16 = false;
  static constexpr bool kIsMax = false;
  static constexpr bool kHasSum = true;
  static constexpr int kPlanes = 2;
  template <int VEC> struct State { float s[VEC]; float c[VEC]; };
  template <int VEC>
  static __device__ __forceinline__ void init(State<VEC>& x) {
#pragma unroll
    for (int k = 0; k < VEC; ++k) { x.s[k] = 0.f; x.c[k] = 0.f; }
  }
  // Knuth's TwoSum: t + e == s + v exactly, whatever the magnitudes.
  static __device__ __forceinline__ void two_sum(float s, float v, float& t, float& e) {
    t = s + v;
    const float bp = t - s;
    e = (s - (t - bp)) + (v - bp);
  }
  // The same TwoSum on two channels at once with the packed fp32x2 instructions of
  // sm_100 (each half rounds exactly like the scalar instruction, so the result is
  // bit-identical); a - b is written fma(b, -1, a), which rounds a - b once.
  static __device__ __forceinline__ void two_sum2(float2 s, float2 v, float2& t, float2& e) {
    const float2 m1 = make_float2(-1.f, -1.f);
    t = __fadd2_rn(s, v);
    const float2 bp = __ffma2_rn(s, m1, t);                 // t - s
    const float2 a = __ffma2_rn(__ffma2_rn(bp, m1, t), m1, s);  // s - (t - bp)
    e = __fadd2_rn(a, __ffma2_rn(bp, m1, v));               // + (v - bp)
  }
  template <int VEC>
  static __device__ __forceinline__ void add(State<VEC>& x, const float (&v)[VEC], int) {
#if TEXB_PACKED_F32X2
    if constexpr (VEC % 2 == 0) {
#pragma unroll
      for (int k = 0; k < VEC; k += 2) {
        float2 t, e;
        two_sum2(make_float2(x.s[k], x.s[k + 1]), make_float2(v[k], v[k + 1]), t, e);
        const float2 c = __fadd2_rn(make_float2(x.c[k], x.c[k + 1]), e);
        x.s[k] = t.x; x.s[k + 1] = t.y;
        x.c[k] = c.x; x.c[k + 1] = c.y;
      }
      return;
    }
#endif
#pragma unroll
    for (int k = 0; k < VEC; ++k) {
      float t, e;
      two_sum(x.s[k], v[k], t, e);
      x.c[k] += e;
      x.s[k] = t;
    }
  }
  template <int VEC>
  static __device__ __forceinline__ void merge(State<VEC>& x, const State<VEC>& y) {
#pragma unroll
    for (int k = 0; k < VEC; ++k) {
      float t, e;
      two_sum(x.s[k], y.s[k], t, e);
      x.c[k] = (x.c[k] + y.c[k]) + e;
      x.s[k] = t;
    }
  }
  template <int VEC>
  static __device__ __forceinline__ void pack(const State<VEC>& x, uint32_t (&w)[kPlanes][VEC]) {
#pragma unroll
    for (int k = 0; k < VEC; ++k) { w[0][k] = __float_as_uint(x.s[k]); w[1][k] = __float_as_uint(x.c[k]); }
  }
  template <int VEC>
  static __device__ __forceinline__ void unpack(State<VEC>& x, const uint32_t (&w)[kPlanes][VEC]) {
#pragma unroll
    for (int k = 0; k < VEC; ++k) { x.s[k] = __uint_as_float(w[0][k]); x.c[k] = __uint_as_float(w[1][k]); }
  }
  // An infinite running sum (infinite input or fp32 overflow) makes the error
  // term NaN; the sum itself is then the answer, as for a plain fp32 sum.
  template <int VEC>
  static __device__ __forceinline__ float value(const State<VEC>& x, int k) {
    return (fabsf(x.s[k]) == INFINITY) ? x.s[k] : x.s[k] + x.c[k];
  }
  template <int VEC>
  static __device__ __forceinline__ float sum_value(const State<VEC>& x, int k) { return value<VEC>(x, k); }
  template <int VEC>
  static __device__ __forceinline__ int index(const State<VEC>&, int) { return 0; }
};

struct OpSumPlain {  // plain fp32 running sum (the "compensated" knob set to 0)
  static constexpr bool kRawBf16 = false;
  static constexpr bool kIsMax = false;
  static constexpr bool kHasSum = true;
  static constexpr int kPlanes = 2;
  template <int VEC> struct State { float s[VEC]; };
  template <int VEC>
  static __device__ __forceinline__ void init(State<VEC>& x) {
#pragma unroll
    for (int k = 0; k < VEC; ++k) x.s[k] = 0.f;
  }
  template <int VEC>
  static __device__ __forceinline__ void add(State<VEC>& x, const float (&v)[VEC], int) {
#pragma unroll
    for (int k = 0; k < VEC; ++k) x.s[k] += v[k];
  }
  template <int VEC>
  static __device__ __forceinline__ void merge(State<VEC>& x, const State<VEC>& y) {
#pragma unroll
    for (int k = 0; k < VEC; ++k) x.s[k] += y.s[k];
  }
  template <int VEC>
  static __device__ __forceinline__ void pack(const State<VEC>& x, uint32_t (&w)[kPlanes][VEC]) {
#pragma unroll
    for (int k = 0; k < VEC; ++k) { w[0][k] = __float_as_uint(x.s[k]); w[1][k] = 0u; }
  }
  template <int VEC>
  static __device__ __forceinline__ void unpack(State<VEC>& x, const uint32_t (&w)[kPlanes][VEC]) {
#pragma unroll
    for (int k = 0; k < VEC; ++k) x.s[k] = __uint_as_float(w[0][k]);
  }
  template <int VEC>
  static __device__ __forceinline__ float value(const State<VEC>& x, int k) { return x.s[k]; }
  template <int VEC>
  static __device__ __forceinline__ float sum_value(const State<VEC>& x, int k) { return x.s[k]; }
  template <int VEC>
  static __device__ __forceinline__ int index(const State<VEC>&, int) { return 0; }
};

// Maximum + row.  Rows reach `add` and pieces reach `merge` in increasing row
// order within a segment (the plan's permutation is stable), so a strict ">"
// keeps the lowest row on ties.  The running value starts at -inf so that a row
// equal to -FLT_MAX still records its index, like the reference's ">=" against
// its -FLT_MAX start (scatter_kernel.cu:139-151); a channel no row claimed
// reports -FLT_MAX / -1, the reference's untouched state.  NaN and -inf never win.
struct OpMax {
  static constexpr bool kRawBf16 = false;
  static constexpr bool kIsMax = true;
  static constexpr bool kHasSum = false;
  static constexpr int kPlanes = 2;
  template <int VEC> struct State { float v[VEC]; int i[VEC]; };
  template <int VEC>
  static __device__ __forceinline__ void init(State<VEC>& x) {
#pragma unroll
    for (int k = 0; k < VEC; ++k) { x.v[k] = -INFINITY; x.i[k] = -1; }
  }
  template <int VEC>
  static __device__ __forceinline__ void add(State<VEC>& x, const float (&v)[VEC], int row) {
#pragma unroll
    for (int k = 0; k < VEC; ++k)
      if (v[k] > x.v[k]) { x.v[k] = v[k]; x.i[k] = row; }
  }
  template <int VEC>
  static __device__ __forceinline__ void merge(State<VEC>& x, const State<VEC>& y) {
#pragma unroll
    for (int k = 0; k < VEC; ++k)
      if (y.v[k] > x.v[k]) { x.v[k] = y.v[k]; x.i[k] = y.i[k]; }
  }
  template <int VEC>
  static __device__ __forceinline__ void pack(const State<VEC>& x, uint32_t (&w)[kPlanes][VEC]) {
#pragma unroll
    for (int k = 0; k < VEC; ++k) { w[0][k] = __float_as_uint(x.v[k]); w[1][k] = uint32_t(x.i[k]); }
  }
  template <int VEC>
  static __device__ __forceinline__ void unpack(State<VEC>& x, const uint32_t (&w)[kPlanes][VEC]) {
#pragma unroll
    for (int k = 0; k < VEC; ++k) { x.v[k] = __uint_as_float(w[0][k]); x.i[k] = int(w[1][k]); }
  }
  template <int VEC>
  static __device__ __forceinline__ float value(const State<VEC>& x, int k) {
    return x.i[k] < 0 ? -FLT_MAX : x.v[k];
  }
  template <int VEC>
  static __device__ __forceinline__ int index(const State<VEC>& x, int k) { return x.i[k]; }
};

// Maximum + row for bf16 rows, kept on packed bf16 pairs: one packed maximum, one packed
// compare (two predicates) and two selects per PAIR of channels instead of unpacking each
// value to fp32 and spending a compare and two selects on it -- the fp32 form keeps the
// integer / logic pipe two thirds busy on 256-byte rows.  Comparisons of bf16 values are
// exact, so the result is the same: strict ">" keeps the lowest row on ties, NaN never
// wins (the packed maximum returns the other operand), -inf never claims a row.  States
// travel through shared memory and the workspace in the same two planes as OpMax
// (fp32 value, row), so stitching and the fix-up are unchanged.
struct OpMaxBf16 {
  static constexpr bool kIsMax = true;
  static constexpr bool kHasSum = false;
  static constexpr int kPlanes = 2;
  static constexpr bool kRawBf16 = true;  // add_raw takes the bf16 pairs as they come from memory
  template <int VEC> struct State { uint32_t b[VEC / 2]; int i[VEC]; };
  template <int VEC>
  static __device__ __forceinline__ void init(State<VEC>& x) {
    static_assert(VEC % 2 == 0, "bf16 channels come in pairs");
#pragma unroll
    for (int j = 0; j < VEC / 2; ++j) x.b[j] = 0xFF80FF80u;  // (-inf, -inf)
#pragma unroll
    for (int k = 0; k < VEC; ++k) x.i[k] = -1;
  }
  // One pair: the low half is the even channel.
  static __device__ __forceinline__ void pair_step(uint32_t& best, int& i_lo, int& i_hi, uint32_t w, int r_lo, int r_hi) {
    asm("{\n"
        ".reg .pred p, q;\n"
        "setp.gt.bf16x2 p|q, %3, %0;\n"
        "max.bf16x2 %0, %0, %3;\n"
        "selp.s32 %1, %4, %1, p;\n"
        "selp.s32 %2, %5, %2, q;\n"
        "}\n"
        : "+r"(best), "+r"(i_lo), "+r"(i_hi) : "r"(w), "r"(r_lo), "r"(r_hi));
  }
  template <int VEC>
  static __device__ __forceinline__ void add_raw(State<VEC>& x, const uint32_t (&w)[VEC / 2], int row) {
#pragma unroll
    for (int j = 0; j < VEC / 2; ++j) pair_step(x.b[j], x.i[2 * j], x.i[2 * j + 1], w[j], row, row);
  }
  // fp32 values that came from bf16 (their low 16 bits are zero): repacked exactly.
  template <int VEC>
  static __device__ __forceinline__ void add(State<VEC>& x, const float (&v)[VEC], int row) {
    uint32_t w[VEC / 2];
#pragma unroll
    for (int j = 0; j < VEC / 2; ++j)
      w[j] = (__float_as_uint(v[2 * j]) >> 16) | (__float_as_uint(v[2 * j + 1]) & 0xffff0000u);
    add_raw<VEC>(x, w, row);
  }
  template <int VEC>
  static __device__ __forceinline__ void merge(State<VEC>& x, const State<VEC>& y) {
#pragma unroll
    for (int j = 0; j < VEC / 2; ++j) pair_step(x.b[j], x.i[2 * j], x.i[2 * j + 1], y.b[j], y.i[2 * j], y.i[2 * j + 1]);
  }
  template <int VEC>
  static __device__ __forceinline__ void pack(const State<VEC>& x, uint32_t (&w)[kPlanes][VEC]) {
#pragma unroll
    for (int j = 0; j < VEC / 2; ++j) {
      w[0][2 * j] = x.b[j] << 16;
      w[0][2 * j + 1] = x.b[j] & 0xffff0000u;
    }
#pragma unroll
    for (int k = 0; k < VEC; ++k) w[1][k] = uint32_t(x.i[k]);
  }
  template <int VEC>
  static __device__ __forceinline__ void unpack(State<VEC>& x, const uint32_t (&w)[kPlanes][VEC]) {
#pragma unroll
    for (int j = 0; j < VEC / 2; ++j) x.b[j] = (w[0][2 * j] >> 16) | (w[0][2 * j + 1] & 0xffff0000u);
#pragma unroll
    for (int k = 0; k < VEC; ++k) x.i[k] = int(w[1][k]);
  }
  template <int VEC>
  static __device__ __forceinline__ float value(const State<VEC>& x, int k) {
    const uint32_t bits = (k & 1) ? (x.b[k / 2] & 0xffff0000u) : (x.b[k / 2] << 16);
    return x.i[k] < 0 ? -FLT_MAX : __uint_as_float(bits);
  }
  template <int VEC>
  static __device__ __forceinline__ int index(const State<VEC>& x, int k) { return x.i[k]; }
};

// Sum (compensated) and maximum + row of the same rows in one pass: the state is
// the two states side by side, and every step is the two operators' step.
struct OpSumMax {
  static constexpr bool kRawBf16 = false;
  static constexpr bool kIsMax = true;
  static constexpr bool kHasSum = true;
  static constexpr int kPlanes = 4;
  template <int VEC> struct State {
    OpSumComp::State<VEC> sum;
    OpMax::State<VEC> max;
  };
  template <int VEC>
  static __device__ __forceinline__ void init(State<VEC>& x) {
    OpSumComp::init<VEC>(x.sum);
    OpMax::init<VEC>(x.max);
  }
  template <int VEC>
  static __device__ __forceinline__ void add(State<VEC>& x, const float (&v)[VEC], int row) {
    OpSumComp::add<VEC>(x.sum, v, row);
    OpMax::add<VEC>(x.max, v, row);
  }
  template <int VEC>
  static __device__ __forceinline__ void merge(State<VEC>& x, const State<VEC>& y) {
    OpSumComp::merge<VEC>(x.sum, y.sum);
    OpMax::merge<VEC>(x.max, y.max);
  }
  template <int VEC>
  static __device__ __forceinline__ void pack(const State<VEC>& x, uint32_t (&w)[kPlanes][VEC]) {
#pragma unroll
    for (int k = 0; k < VEC; ++k) {
      w[0][k] = __float_as_uint(x.sum.s[k]); w[1][k] = __float_as_uint(x.sum.c[k]);
      w[2][k] = __float_as_uint(x.max.v[k]); w[3][k] = uint32_t(x.max.i[k]);
    }
  }
  template <int VEC>
  static __device__ __forceinline__ void unpack(State<VEC>& x, const uint32_t (&w)[kPlanes][VEC]) {
#pragma unroll
    for (int k = 0; k < VEC; ++k) {
      x.sum.s[k] = __uint_as_float(w[0][k]); x.sum.c[k] = __uint_as_float(w[1][k]);
      x.max.v[k] = __uint_as_float(w[2][k]); x.max.i[k] = int(w[3][k]);
    }
  }
  template <int VEC>
  static __device__ __forceinline__ float value(const State<VEC>& x, int k) { return OpMax::value<VEC>(x.max, k); }
  template <int VEC>
  static __device__ __forceinline__ int index(const State<VEC>& x, int k) { return x.max.i[k]; }
  template <int VEC>
  static __device__ __forceinline__ float sum_value(const State<VEC>& x, int k) { return OpSumComp::value<VEC>(x.sum, k); }
};

}  // namespace texb
