// Helpers shared by the write-law kernels (refine.cu, refine_mrk.cu): 8-wide vector loads / stores,
// the row's 1/rms from the per-head sums of squares, and the thread -> (row, head, rotation pairs) map.
// One thread owns 8 adjacent rotation pairs of one head: columns [c0, c0+8) and [c0+half, c0+half+8),
// so every access is a 16-byte vector; the DH/16 threads of a head are adjacent lanes of one warp.
#pragma once
#include "common.cuh"

namespace {

struct V8 {
  float x[8];
};
__device__ __forceinline__ V8 ld8(const bf16* p) {
  uint4 u = *reinterpret_cast<const uint4*>(p);
  float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y), c = unpack_bf16(u.z), d = unpack_bf16(u.w);
  return V8{{a.x, a.y, b.x, b.y, c.x, c.y, d.x, d.y}};
}
__device__ __forceinline__ void st8(bf16* p, const V8& v) {
  *reinterpret_cast<uint4*>(p) = make_uint4(pack_bf16(v.x[0], v.x[1]), pack_bf16(v.x[2], v.x[3]),
                                            pack_bf16(v.x[4], v.x[5]), pack_bf16(v.x[6], v.x[7]));
}
__device__ __forceinline__ V8 ld8f(const float* p) {
  float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  return V8{{a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w}};
}
__device__ __forceinline__ void st8f(float* p, const V8& v) {
  *reinterpret_cast<float4*>(p) = make_float4(v.x[0], v.x[1], v.x[2], v.x[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(v.x[4], v.x[5], v.x[6], v.x[7]);
}
__device__ __forceinline__ void acc8f(float* p, const V8& v) {
  V8 o = ld8f(p);
#pragma unroll
  for (int i = 0; i < 8; ++i) o.x[i] += v.x[i];
  st8f(p, o);
}
// the row's 1/rms from its H per-head sums of squares: 16-byte loads when the head count keeps the rows
// 16-byte aligned, scalar loads otherwise (e.g. 15 heads)
__device__ __forceinline__ float row_rstd(const float* ssq_row, int H, int d, float eps) {
  float s = 0.f;
  if ((H & 3) == 0) {
    for (int i = 0; i < H; i += 4) {
      float4 v = *reinterpret_cast<const float4*>(ssq_row + i);
      s += v.x + v.y + v.z + v.w;
    }
  } else {
    for (int i = 0; i < H; ++i) s += ssq_row[i];
  }
  return rsqrtf(s / d + eps);
}

struct Where {
  long long row;   // b * C + t
  int b, t, c0, c1; // chunk-local position and this thread's two column bases
  int p0;          // first rotation pair index inside the head
};
__device__ __forceinline__ bool locate(Where& w, long long i, int B, int C, int H, int DH) {
  const int half = DH >> 1, per_head = half >> 3;   // threads per head
  const long long total = (long long)B * C * H * per_head;
  if (i >= total) return false;
  const int q = i % per_head;
  long long r = i / per_head;
  const int h = r % H;
  r /= H;
  w.t = r % C;
  w.b = r / C;
  w.row = (long long)w.b * C + w.t;
  w.p0 = q * 8;
  w.c0 = h * DH + w.p0;
  w.c1 = w.c0 + half;
  return true;
}

// sum over the threads of one head (DH/16 adjacent lanes; a power of two <= 32)
__device__ __forceinline__ float head_sum(float v, int per_head) {
  for (int o = per_head >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

}  // namespace
