// Single-token decode read over the recurrent KV tape.
//
// One CTA per (batch row, head).  The tape is [B, P, H, DH] bf16 with `*pos_ptr` live rows; the
// position is read from device memory so the launch can sit inside a CUDA graph that is replayed
// for every token.  Only the live rows (and, with a sliding window, only the last W-1 of them)
// are read - the kernel is a pure HBM stream of K and V with an online softmax - and the
// position's own RAW key/value enter as one extra softmax column.
#include "common.cuh"

namespace {

constexpr int DEC_WARPS = 8;        // 8 warps x 4 key steps x 32 bytes of K and of V in flight per thread

template <int DH>
__global__ void __launch_bounds__(DEC_WARPS * 32) decode_attend_kernel(
    const bf16* __restrict__ q, const bf16* __restrict__ kself, const bf16* __restrict__ vself,
    const bf16* __restrict__ K, const bf16* __restrict__ V, const int* __restrict__ pos_ptr,
    bf16* __restrict__ out, float* __restrict__ ssq, int P, int H, float scale, int window) {
  constexpr int LPK = DH / 8;        // lanes per key (each lane owns 8 contiguous dims)
  constexpr int KPW = 32 / LPK;      // keys per warp step
  constexpr int NW = DEC_WARPS;
  __shared__ float s_m[NW * KPW], s_l[NW * KPW];
  __shared__ float s_acc[NW * KPW][DH];
  __shared__ float s_sq[DH / 32];
  const int h = blockIdx.x, b = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int grp = lane / LPK, sub = lane % LPK;
  const int pos = *pos_ptr;                       // rows [0, pos) are live
  const int lo = window > 0 ? max(0, pos - (window - 1)) : 0;
  const long long row_stride = (long long)H * DH;
  const bf16* Kb = K + ((long long)b * P) * row_stride + (long long)h * DH + sub * 8;
  const bf16* Vb = V + ((long long)b * P) * row_stride + (long long)h * DH + sub * 8;
  const long long qoff = ((long long)b * H + h) * DH + sub * 8;
  float qv[8];
  {
    uint4 u = *reinterpret_cast<const uint4*>(q + qoff);
    float2 a = unpack_bf16(u.x), c = unpack_bf16(u.y), e = unpack_bf16(u.z), f = unpack_bf16(u.w);
    qv[0] = a.x; qv[1] = a.y; qv[2] = c.x; qv[3] = c.y; qv[4] = e.x; qv[5] = e.y; qv[6] = f.x; qv[7] = f.y;
  }
  float m = -INFINITY, l = 0.f, acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;
  // the loop bound is warp-uniform (all lanes run the shuffles); a group past the end is masked.
  // U key steps per iteration: all their loads are issued before the first use, so every thread keeps
  // U x 32 bytes in flight (the kernel is a pure HBM stream; one step at a time left the bus half idle)
  constexpr int U = 4;
  for (int j0 = lo + warp * KPW; j0 < pos; j0 += U * NW * KPW) {
    uint4 ku[U], vu[U];
    bool live[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int j = j0 + u * NW * KPW + grp;
      live[u] = j < pos;
      ku[u] = make_uint4(0, 0, 0, 0);
      vu[u] = make_uint4(0, 0, 0, 0);
      if (live[u]) {
        ku[u] = *reinterpret_cast<const uint4*>(Kb + (long long)j * row_stride);
        vu[u] = *reinterpret_cast<const uint4*>(Vb + (long long)j * row_stride);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      float2 k0 = unpack_bf16(ku[u].x), k1 = unpack_bf16(ku[u].y), k2 = unpack_bf16(ku[u].z), k3 = unpack_bf16(ku[u].w);
      float s = qv[0] * k0.x + qv[1] * k0.y + qv[2] * k1.x + qv[3] * k1.y + qv[4] * k2.x + qv[5] * k2.y +
                qv[6] * k3.x + qv[7] * k3.y;
#pragma unroll
      for (int o = LPK / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
      s *= scale;
      if (!live[u]) continue;
      const float mn = fmaxf(m, s), c = __expf(m - mn), p = __expf(s - mn);
      float2 v0 = unpack_bf16(vu[u].x), v1 = unpack_bf16(vu[u].y), v2 = unpack_bf16(vu[u].z), v3 = unpack_bf16(vu[u].w);
      l = l * c + p;
      acc[0] = acc[0] * c + p * v0.x; acc[1] = acc[1] * c + p * v0.y;
      acc[2] = acc[2] * c + p * v1.x; acc[3] = acc[3] * c + p * v1.y;
      acc[4] = acc[4] * c + p * v2.x; acc[5] = acc[5] * c + p * v2.y;
      acc[6] = acc[6] * c + p * v3.x; acc[7] = acc[7] * c + p * v3.y;
      m = mn;
    }
  }
  const int slot = warp * KPW + grp;
  if (sub == 0) { s_m[slot] = m; s_l[slot] = l; }
#pragma unroll
  for (int i = 0; i < 8; ++i) s_acc[slot][sub * 8 + i] = acc[i];
  __syncthreads();
  // final merge: thread t < DH owns output dim t
  const int t = threadIdx.x;
  if (t < DH) {
    const long long so = ((long long)b * H + h) * DH;
    // raw self column
    float ss = 0.f;
    for (int d = 0; d < DH; ++d) ss += __bfloat162float(q[so + d]) * __bfloat162float(kself[so + d]);
    ss *= scale;
    float M = ss;
    for (int s = 0; s < NW * KPW; ++s) M = fmaxf(M, s_m[s]);
    float Z = __expf(ss - M), o = Z * __bfloat162float(vself[so + t]);
    for (int s = 0; s < NW * KPW; ++s) {
      const float w = s_l[s] > 0.f ? __expf(s_m[s] - M) : 0.f;
      Z += w * s_l[s];
      o += w * s_acc[s][t];
    }
    const float val = o / Z;
    out[so + t] = __float2bfloat16(val);
    if (ssq) {                                     // sum of squares of the head's read (the row norm of the write law)
      float sq = val * val;
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, off);
      if (lane == 0) s_sq[warp] = sq;
    }
  }
  if (ssq) {
    __syncthreads();
    if (t == 0) {
      float tot = 0.f;
      for (int w = 0; w < DH / 32; ++w) tot += s_sq[w];
      ssq[(long long)b * H + h] = tot;
    }
  }
}

}  // namespace

extern "C" {

// q, kself, vself, out: [B, H, DH] bf16 contiguous; K, V: [B, P, H, DH] bf16 contiguous; ssq: optional [B, H] fp32
// (sum over the head's dims of out^2).
int dmb_decode_attend(const void* q, const void* kself, const void* vself, const void* K, const void* V,
                      const int* pos_ptr, void* out, float* ssq, int B, int P, int H, int dh, float scale, int window,
                      cudaStream_t st) {
  dim3 grid(H, B);
  if (dh == 64)
    decode_attend_kernel<64><<<grid, DEC_WARPS * 32, 0, st>>>((const bf16*)q, (const bf16*)kself, (const bf16*)vself, (const bf16*)K, (const bf16*)V, pos_ptr, (bf16*)out, ssq, P, H, scale, window);
  else if (dh == 128)
    decode_attend_kernel<128><<<grid, DEC_WARPS * 32, 0, st>>>((const bf16*)q, (const bf16*)kself, (const bf16*)vself, (const bf16*)K, (const bf16*)V, pos_ptr, (bf16*)out, ssq, P, H, scale, window);
  else
    return -1;
  DMB_CHECK_LAUNCH();
  return 0;
}

}  // extern "C"
