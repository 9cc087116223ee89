// Four-channel helpers used by the generated channelwise bodies (generated/cw_groups.cuh).
// A thread owns four consecutive channels; a[4] is one value per channel.
#pragma once

#define CW_MUL4(d, s, a)                                                        \
  { d[0] = (s) * a[0]; d[1] = (s) * a[1]; d[2] = (s) * a[2]; d[3] = (s) * a[3]; }
#define CW_FMA4(d, s, a)                                                        \
  { d[0] = fmaf((s), a[0], d[0]); d[1] = fmaf((s), a[1], d[1]);                  \
    d[2] = fmaf((s), a[2], d[2]); d[3] = fmaf((s), a[3], d[3]); }
#define CW_MULV4(d, a, b)                                                       \
  { d[0] = a[0] * b[0]; d[1] = a[1] * b[1]; d[2] = a[2] * b[2]; d[3] = a[3] * b[3]; }
#define CW_FMAV4(d, a, b)                                                       \
  { d[0] = fmaf(a[0], b[0], d[0]); d[1] = fmaf(a[1], b[1], d[1]);                \
    d[2] = fmaf(a[2], b[2], d[2]); d[3] = fmaf(a[3], b[3], d[3]); }
#define CW_DOT4(a, b) fmaf(a[3], b[3], fmaf(a[2], b[2], fmaf(a[1], b[1], a[0] * b[0])))

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
