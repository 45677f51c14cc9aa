// Shared pieces of the chunk-cell attention kernels: padded shared-memory tiles, ldmatrix
// fragment loaders for the four operand orientations, tile copies and quad dot products.
#pragma once
#include "common.cuh"

namespace attn {

template <int DH>
struct Tile {
  static constexpr int PITCH = DH + 8;  // +16 B per row: conflict-free ldmatrix
};

// ---- fragment loaders --------------------------------------------------------------------
template <int PITCH>
__device__ __forceinline__ void load_a(uint32_t (&a)[4], const bf16* t, int row0, int k0, int lane) {
  int r = row0 + (lane & 15), c = k0 + ((lane >> 4) << 3);
  ldsm_x4(a[0], a[1], a[2], a[3], smem_u32(t + r * PITCH + c));
}
// B for n-blocks [n0, n0+16) x k [k0, k0+16) from a tile stored [n][k]
template <int PITCH>
__device__ __forceinline__ void load_b_nk(uint32_t (&b)[4], const bf16* t, int n0, int k0, int lane) {
  int n = n0 + (lane & 7) + ((lane >> 4) << 3), k = k0 + (((lane >> 3) & 1) << 3);
  ldsm_x4(b[0], b[1], b[2], b[3], smem_u32(t + n * PITCH + k));
}
// B for k [k0, k0+16) x n-blocks [n0, n0+16) from a tile stored [k][n]
template <int PITCH>
__device__ __forceinline__ void load_b_kn(uint32_t (&b)[4], const bf16* t, int k0, int n0, int lane) {
  int k = k0 + (lane & 7) + (((lane >> 3) & 1) << 3), n = n0 + ((lane >> 4) << 3);
  ldsm_x4_t(b[0], b[1], b[2], b[3], smem_u32(t + k * PITCH + n));
}
// A = X^T block (m [m0,m0+16), k [k0,k0+16)) from X stored [k][m]
template <int PITCH>
__device__ __forceinline__ void load_a_t(uint32_t (&a)[4], const bf16* t, int m0, int k0, int lane) {
  int i = lane >> 3;
  int r = k0 + (lane & 7) + ((i >> 1) << 3), c = m0 + ((i & 1) << 3);
  ldsm_x4_t(a[0], a[1], a[2], a[3], smem_u32(t + r * PITCH + c));
}

// rows x DH bf16 from global (row stride rs elements) into a padded tile
template <int DH, int NT>
__device__ __forceinline__ void load_tile_bf16(bf16* dst, const bf16* src, long long rs, int rows,
                                               int tid) {
  constexpr int P = Tile<DH>::PITCH, CH = DH / 8;
  for (int i = tid; i < rows * CH; i += NT) {
    int r = i / CH, c = (i % CH) * 8;
    *reinterpret_cast<uint4*>(dst + r * P + c) = *reinterpret_cast<const uint4*>(src + r * rs + c);
  }
}
template <int DH, int NT>
__device__ __forceinline__ void load_tile_f32(bf16* dst, const float* src, long long rs, int rows,
                                              int tid) {
  constexpr int P = Tile<DH>::PITCH, CH = DH / 4;
  for (int i = tid; i < rows * CH; i += NT) {
    int r = i / CH, c = (i % CH) * 4;
    float4 v = *reinterpret_cast<const float4*>(src + r * rs + c);
    uint2 u = make_uint2(pack_bf16(v.x, v.y), pack_bf16(v.z, v.w));
    *reinterpret_cast<uint2*>(dst + r * P + c) = u;
  }
}
template <int DH, int NT>
__device__ __forceinline__ void load_tile_async(bf16* dst, const bf16* src, long long rs, int rows,
                                                int tid) {
  constexpr int P = Tile<DH>::PITCH, CH = DH / 8;
  for (int i = tid; i < rows * CH; i += NT) {
    int r = i / CH, c = (i % CH) * 8;
    cp_async16(dst + r * P + c, src + r * rs + c);
  }
}

// per-row dot product of two DH-vectors split over the 4 lanes of a quad: lane t takes the contiguous
// elements [t * DH/4, (t+1) * DH/4) with 16-byte loads (both rows must be 16-byte aligned: they are rows
// of head slices of tensors whose head dim is a multiple of 32)
__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  float2 a = __bfloat1622float2(*reinterpret_cast<const bf162*>(&u.x));
  float2 b = __bfloat1622float2(*reinterpret_cast<const bf162*>(&u.y));
  float2 c = __bfloat1622float2(*reinterpret_cast<const bf162*>(&u.z));
  float2 d = __bfloat1622float2(*reinterpret_cast<const bf162*>(&u.w));
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
template <int DH>
__device__ __forceinline__ float quad_dot_bf16(const bf16* a, const bf16* b, int t) {
  constexpr int PER = DH / 4;
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < PER / 8; ++i) {
    float x[8], y[8];
    unpack8(*reinterpret_cast<const uint4*>(a + t * PER + 8 * i), x);
    unpack8(*reinterpret_cast<const uint4*>(b + t * PER + 8 * i), y);
#pragma unroll
    for (int e = 0; e < 8; ++e) s += x[e] * y[e];
  }
  return quad_sum(s);
}
template <int DH>
__device__ __forceinline__ float quad_dot_f32_bf16(const float* a, const bf16* b, int t) {
  constexpr int PER = DH / 4;
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < PER / 8; ++i) {
    float y[8];
    const float4 x0 = *reinterpret_cast<const float4*>(a + t * PER + 8 * i);
    const float4 x1 = *reinterpret_cast<const float4*>(a + t * PER + 8 * i + 4);
    unpack8(*reinterpret_cast<const uint4*>(b + t * PER + 8 * i), y);
    s += x0.x * y[0] + x0.y * y[1] + x0.z * y[2] + x0.w * y[3] + x1.x * y[4] + x1.y * y[5] + x1.z * y[6] + x1.w * y[7];
  }
  return quad_sum(s);
}
template <int DH>
__device__ __forceinline__ float quad_dot_f32(const float* a, const float* b, int t) {
  constexpr int PER = DH / 4;
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < PER / 4; ++i) {
    const float4 x = *reinterpret_cast<const float4*>(a + t * PER + 4 * i);
    const float4 y = *reinterpret_cast<const float4*>(b + t * PER + 4 * i);
    s += x.x * y.x + x.y * y.y + x.z * y.z + x.w * y.w;
  }
  return quad_sum(s);
}

__device__ __forceinline__ bool intra_ok(int i, int j, int window) {
  return j < i && (window == 0 || j > i - window);
}

constexpr int KT = 64;  // keys per tile of the prefix passes

template <typename K>
int set_smem(K kernel, size_t bytes) {
  if (bytes > 48 * 1024)
    return (int)cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
  return 0;
}

}  // namespace attn

#define DISPATCH_DH_C(DH_, C_, ...)                                   \
  if (DH_ == 64 && C_ == 16) { constexpr int DH = 64, C = 16; __VA_ARGS__ }   \
  else if (DH_ == 64 && C_ == 32) { constexpr int DH = 64, C = 32; __VA_ARGS__ }   \
  else if (DH_ == 64 && C_ == 64) { constexpr int DH = 64, C = 64; __VA_ARGS__ }   \
  else if (DH_ == 128 && C_ == 16) { constexpr int DH = 128, C = 16; __VA_ARGS__ } \
  else if (DH_ == 128 && C_ == 32) { constexpr int DH = 128, C = 32; __VA_ARGS__ } \
  else if (DH_ == 128 && C_ == 64) { constexpr int DH = 128, C = 64; __VA_ARGS__ } \
  else return -1;
