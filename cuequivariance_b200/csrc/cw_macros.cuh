// Per-thread channel-vector helpers used by the generated channelwise bodies
// (generated/cw_groups.cuh).  A thread owns C consecutive channels (C = 2 or 4); a[C] holds
// one value per channel.
#pragma once

template <int C>
__device__ __forceinline__ void cw_mul(float (&d)[C], float s, const float (&a)[C]) {
#pragma unroll
  for (int c = 0; c < C; ++c) d[c] = s * a[c];
}
template <int C>
__device__ __forceinline__ void cw_fma(float (&d)[C], float s, const float (&a)[C]) {
#pragma unroll
  for (int c = 0; c < C; ++c) d[c] = fmaf(s, a[c], d[c]);
}
template <int C>
__device__ __forceinline__ void cw_mulv(float (&d)[C], const float (&a)[C], const float (&b)[C]) {
#pragma unroll
  for (int c = 0; c < C; ++c) d[c] = a[c] * b[c];
}
template <int C>
__device__ __forceinline__ void cw_fmav(float (&d)[C], const float (&a)[C], const float (&b)[C]) {
#pragma unroll
  for (int c = 0; c < C; ++c) d[c] = fmaf(a[c], b[c], d[c]);
}
template <int C>
__device__ __forceinline__ float cw_dot(const float (&a)[C], const float (&b)[C]) {
  float v = a[0] * b[0];
#pragma unroll
  for (int c = 1; c < C; ++c) v = fmaf(a[c], b[c], v);
  return v;
}
#define CW_MUL4(d, s, a) cw_mul(d, s, a)
#define CW_FMA4(d, s, a) cw_fma(d, s, a)
#define CW_MULV4(d, a, b) cw_mulv(d, a, b)
#define CW_FMAV4(d, a, b) cw_fmav(d, a, b)
#define CW_DOT4(a, b) cw_dot(a, b)

// Loads N consecutive floats starting at M[Q0] (M is 16-byte aligned shared memory, every
// lane reads the same addresses: broadcast) using 128-bit loads where the alignment allows.
template <int Q0, int N>
__device__ __forceinline__ void cw_load_m(const float* __restrict__ M, float (&m)[N]) {
  constexpr int A0 = Q0 & ~3;                 // first aligned float4
  constexpr int A1 = (Q0 + N + 3) & ~3;       // one past the last
#pragma unroll
  for (int a = A0; a < A1; a += 4) {
    const float4 v = *reinterpret_cast<const float4*>(M + a);
    if (a + 0 >= Q0 && a + 0 < Q0 + N) m[a + 0 - Q0] = v.x;
    if (a + 1 >= Q0 && a + 1 < Q0 + N) m[a + 1 - Q0] = v.y;
    if (a + 2 >= Q0 && a + 2 < Q0 + N) m[a + 2 - Q0] = v.z;
    if (a + 3 >= Q0 && a + 3 < Q0 + N) m[a + 3 - Q0] = v.w;
  }
}
