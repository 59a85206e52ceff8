// A kernel input that is either a stored matrix (float32 or bfloat16) or the float32
// partial products of a matrix product whose k was split ([splits][n], `stride` elements
// apart), which the reader adds in split order while it loads.  kind: 0 float32 (one or
// several splits), 1 bfloat16.
#pragma once

#include "common.cuh"

struct Source {
  const void* p;
  int kind;
  int splits;
  long long stride;
};

static inline Source make_source(const void* p, int kind, int splits, long long stride) {
  Source s;
  s.p = p;
  s.kind = kind;
  s.splits = splits < 1 ? 1 : splits;
  s.stride = stride;
  return s;
}

__device__ __forceinline__ float source_load(const Source& s, long long i) {
  if (s.kind == 1) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(s.p)[i]);
  const float* f = reinterpret_cast<const float*>(s.p);
  float v = f[i];
  for (int k = 1; k < s.splits; ++k) v = __fadd_rn(v, f[(long long)k * s.stride + i]);
  return v;
}

// Store a float32 value as the dtype code says (0 float32, 1 bfloat16).
__device__ __forceinline__ void store_as(void* p, int dtype, long long i, float v) {
  if (dtype == 1) reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
  else reinterpret_cast<float*>(p)[i] = v;
}
__device__ __forceinline__ float load_as(const void* p, int dtype, long long i) {
  if (dtype == 1) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
  return reinterpret_cast<const float*>(p)[i];
}

__device__ __forceinline__ float sigmoid_f32(float x) { return 1.0f / (1.0f + expf(-x)); }
