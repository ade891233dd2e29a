// Register-tile arithmetic used by kernel epilogues: casts, element-wise maps,
// reductions.  The reference exposes these as tile_cast / tile_elementwise /
// tile_reduce / tile_zeros / tile_full over Triton blocks
// (tileccl/primitives/compute.py:13-179); here a thread's slice of the tile is a
// small array of fp32 registers (one TMEM row segment).  tile_dot has no free
// function: matrix products are issued by the tcgen05 main loop in
// kernels/gemm_sm100.cu.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace tileccl {

enum ElementwiseOp : int {
  kOpIdentity = 0,
  kOpExp = 1,
  kOpLog = 2,
  kOpAbs = 3,
  kOpNeg = 4,
  kOpSqrt = 5,
  kOpRelu = 6,
  kOpSigmoid = 7,
  kOpSilu = 8,
};

__device__ __forceinline__ float apply_elementwise(int op, float x) {
  switch (op) {
    case kOpExp: return __expf(x);
    case kOpLog: return __logf(x);
    case kOpAbs: return fabsf(x);
    case kOpNeg: return -x;
    case kOpSqrt: return sqrtf(x);
    case kOpRelu: return fmaxf(x, 0.f);
    case kOpSigmoid: return 1.f / (1.f + __expf(-x));
    case kOpSilu: return x / (1.f + __expf(-x));
    default: return x;
  }
}

template <int N>
__device__ __forceinline__ void tile_elementwise(int op, float (&v)[N]) {
#pragma unroll
  for (int i = 0; i < N; ++i) v[i] = apply_elementwise(op, v[i]);
}
template <int N>
__device__ __forceinline__ void tile_zeros(float (&v)[N]) {
#pragma unroll
  for (int i = 0; i < N; ++i) v[i] = 0.f;
}
template <int N>
__device__ __forceinline__ void tile_full(float (&v)[N], float x) {
#pragma unroll
  for (int i = 0; i < N; ++i) v[i] = x;
}

// Reduce a thread's fragment, then across the warp.  mode: 0 sum, 1 max, 2 min.
template <int N>
__device__ __forceinline__ float tile_reduce(const float (&v)[N], int mode) {
  float a = v[0];
#pragma unroll
  for (int i = 1; i < N; ++i) a = mode == 0 ? a + v[i] : mode == 1 ? fmaxf(a, v[i]) : fminf(a, v[i]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float b = __shfl_xor_sync(0xffffffffu, a, o);
    a = mode == 0 ? a + b : mode == 1 ? fmaxf(a, b) : fminf(a, b);
  }
  return a;
}

// Pack two fp32 into one 32-bit word of fp16 / bf16 (low half = first value).
__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ uint32_t pack_16x2(bool is_bf16, float lo, float hi) {
  return is_bf16 ? pack_bf16x2(lo, hi) : pack_f16x2(lo, hi);
}
__device__ __forceinline__ float2 unpack_16x2(bool is_bf16, uint32_t w) {
  if (is_bf16) {
    __nv_bfloat162 h = *reinterpret_cast<__nv_bfloat162*>(&w);
    return __bfloat1622float2(h);
  }
  __half2 h = *reinterpret_cast<__half2*>(&w);
  return __half22float2(h);
}

// tile_cast: 8 fp32 -> one 16-byte vector of 16-bit floats.
__device__ __forceinline__ uint4 tile_cast_f32x8(bool is_bf16, const float* v) {
  uint4 o;
  o.x = pack_16x2(is_bf16, v[0], v[1]);
  o.y = pack_16x2(is_bf16, v[2], v[3]);
  o.z = pack_16x2(is_bf16, v[4], v[5]);
  o.w = pack_16x2(is_bf16, v[6], v[7]);
  return o;
}
// acc[0..7] += the eight 16-bit floats in `w`.
__device__ __forceinline__ void tile_accumulate_16x8(bool is_bf16, float* acc, const uint4& w) {
  float2 a = unpack_16x2(is_bf16, w.x), b = unpack_16x2(is_bf16, w.y);
  float2 c = unpack_16x2(is_bf16, w.z), d = unpack_16x2(is_bf16, w.w);
  acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y;
  acc[4] += c.x; acc[5] += c.y; acc[6] += d.x; acc[7] += d.y;
}

}  // namespace tileccl
