// Bandwidth-bound fused kernels: RMSNorm fwd/bwd, RoPE, SwiGLU
// fwd/bwd, the cross-entropy slab (loss + d logits) and column reductions.  All activations are
// bf16, all statistics and gradients of parameters fp32.
#include <stdio.h>

#include "common.cuh"
#include "noalloc.h"

namespace {

// ---- RMSNorm --------------------------------------------------------------------------------
// one warp per row; d % 8 == 0
__global__ void rms_fwd_kernel(const bf16* __restrict__ x, long long xs, const bf16* __restrict__ w,
                               bf16* __restrict__ y, float* __restrict__ rstd, int rows, int d,
                               float eps) {
  int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= rows) return;
  const bf16* xr = x + (long long)row * xs;
  float ss = 0.f;
  for (int c = lane * 8; c < d; c += 256) {
    uint4 u = *reinterpret_cast<const uint4*>(xr + c);
    float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y), e = unpack_bf16(u.z), f = unpack_bf16(u.w);
    ss += a.x * a.x + a.y * a.y + b.x * b.x + b.y * b.y + e.x * e.x + e.y * e.y + f.x * f.x + f.y * f.y;
  }
  ss = warp_sum(ss);
  float r = rsqrtf(ss / d + eps);
  if (lane == 0 && rstd) rstd[row] = r;
  bf16* yr = y + (long long)row * d;
  for (int c = lane * 8; c < d; c += 256) {
    uint4 u = *reinterpret_cast<const uint4*>(xr + c);
    uint4 wv = *reinterpret_cast<const uint4*>(w + c);
    float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y), e = unpack_bf16(u.z), f = unpack_bf16(u.w);
    float2 wa = unpack_bf16(wv.x), wb = unpack_bf16(wv.y), we = unpack_bf16(wv.z), wf = unpack_bf16(wv.w);
    uint4 o;
    o.x = pack_bf16(a.x * r * wa.x, a.y * r * wa.y);
    o.y = pack_bf16(b.x * r * wb.x, b.y * r * wb.y);
    o.z = pack_bf16(e.x * r * we.x, e.y * r * we.y);
    o.w = pack_bf16(f.x * r * wf.x, f.y * r * wf.y);
    *reinterpret_cast<uint4*>(yr + c) = o;
  }
}

template <typename TDY>
__device__ __forceinline__ float ld1(const TDY* p);
template <>
__device__ __forceinline__ float ld1<float>(const float* p) { return *p; }
template <>
__device__ __forceinline__ float ld1<bf16>(const bf16* p) { return __bfloat162float(*p); }

// dx = rstd * (g - xn * mean(g * xn)), g = dy * w, xn = x * rstd; one warp per row, d % 2 == 0.
// out = (residual ? residual : 0) + dx, written as fp32 or bf16.
template <typename TDY, typename TOUT>
__global__ void rms_bwd_dx_kernel(const TDY* __restrict__ dy, const bf16* __restrict__ x, long long xs,
                                  const bf16* __restrict__ w, const float* __restrict__ rstd,
                                  const TOUT* __restrict__ residual, TOUT* __restrict__ out, int rows,
                                  int d) {
  int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= rows) return;
  const bf16* xr = x + (long long)row * xs;
  const TDY* dyr = dy + (long long)row * d;
  const float r = rstd[row];
  float acc = 0.f;
  for (int c = lane; c < d; c += 32)
    acc += ld1(dyr + c) * __bfloat162float(w[c]) * __bfloat162float(xr[c]) * r;
  const float mean = warp_sum(acc) / d;
  for (int c = lane; c < d; c += 32) {
    float xn = __bfloat162float(xr[c]) * r;
    float g = ld1(dyr + c) * __bfloat162float(w[c]);
    float v = r * (g - xn * mean);
    long long o = (long long)row * d + c;
    if (residual) v += ld1(residual + o);
    if constexpr (sizeof(TOUT) == 4) out[o] = v; else out[o] = __float2bfloat16(v);
  }
}

// partial[s][col] = sum over the rows of split s of dy * x * rstd  (rstd == nullptr: plain column sum of dy)
template <typename TDY>
__global__ void col_partial_kernel(const TDY* __restrict__ dy, const bf16* __restrict__ x, long long xs,
                                   const float* __restrict__ rstd, float* __restrict__ partial, int rows,
                                   int d, int rows_per_split) {
  __shared__ float red[8][64];
  const int col = blockIdx.x * 64 + (threadIdx.x & 63), wy = threadIdx.x >> 6;  // 8 row lanes x 64 cols
  const int r0 = blockIdx.y * rows_per_split, r1 = min(rows, r0 + rows_per_split);
  float acc = 0.f;
  if (col < d) {
    for (int r = r0 + wy; r < r1; r += 8) {
      float v = ld1(dy + (long long)r * d + col);
      if (rstd) v *= __bfloat162float(x[(long long)r * xs + col]) * rstd[r];
      acc += v;
    }
  }
  red[wy][threadIdx.x & 63] = acc;
  __syncthreads();
  if (wy == 0 && col < d) {
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) s += red[i][threadIdx.x];
    partial[(long long)blockIdx.y * d + col] = s;
  }
}

__global__ void reduce_partials_kernel(const float* __restrict__ partial, float* __restrict__ out,
                                       int nsplit, int d) {
  int col = blockIdx.x * blockDim.x + threadIdx.x;
  if (col >= d) return;
  float s = 0.f;
  for (int i = 0; i < nsplit; ++i) s += partial[(long long)i * d + col];
  out[col] += s;
}

// ---- RoPE -----------------------------------------------------------------------------------------
// x [B, T, H, DH] with batch stride bs and row stride rs (elements); out contiguous.  sign=-1 inverts.
template <typename TI, typename TO>
__global__ void rope_kernel(const TI* __restrict__ x, long long bs, long long rs,
                            const float* __restrict__ cosb, const float* __restrict__ sinb,
                            TO* __restrict__ out, int B, int T, int H, int DH, float sign) {
  const int half = DH >> 1;
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  long long total = (long long)B * T * H * half;
  if (i >= total) return;
  int p = i % half;
  long long r = i / half;
  int h = r % H;
  r /= H;
  int t = r % T, b = r / T;
  const TI* src = x + b * bs + (long long)t * rs + h * DH;
  float lo = ld1(src + p), hi = ld1(src + p + half);
  float c = cosb[t * half + p], s = sign * sinb[t * half + p];
  long long o = (((long long)b * T + t) * H + h) * DH;
  float a = lo * c - hi * s, bb = hi * c + lo * s;
  if constexpr (sizeof(TO) == 4) { out[o + p] = a; out[o + p + half] = bb; }
  else { out[o + p] = __float2bfloat16(a); out[o + p + half] = __float2bfloat16(bb); }
}

// ---- SwiGLU ---------------------------------------------------------------------------------------------------
__global__ void swiglu_fwd_kernel(const bf16* __restrict__ h1, const bf16* __restrict__ h3,
                                  bf16* __restrict__ g, long long n8) {
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n8) return;
  uint4 a = reinterpret_cast<const uint4*>(h1)[i], b = reinterpret_cast<const uint4*>(h3)[i], o;
  uint32_t* ap = &a.x; uint32_t* bp = &b.x; uint32_t* op = &o.x;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    float2 x = unpack_bf16(ap[j]), y = unpack_bf16(bp[j]);
    op[j] = pack_bf16(x.x * sigmoidf_(x.x) * y.x, x.y * sigmoidf_(x.y) * y.y);
  }
  reinterpret_cast<uint4*>(g)[i] = o;
}

__global__ void swiglu_bwd_kernel(const bf16* __restrict__ dg, const bf16* __restrict__ h1,
                                  const bf16* __restrict__ h3, bf16* __restrict__ dh1,
                                  bf16* __restrict__ dh3, long long n8) {
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n8) return;
  uint4 g = reinterpret_cast<const uint4*>(dg)[i], a = reinterpret_cast<const uint4*>(h1)[i],
        b = reinterpret_cast<const uint4*>(h3)[i], o1, o3;
  uint32_t* gp = &g.x; uint32_t* ap = &a.x; uint32_t* bp = &b.x; uint32_t* p1 = &o1.x; uint32_t* p3 = &o3.x;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    float2 dgv = unpack_bf16(gp[j]), x = unpack_bf16(ap[j]), y = unpack_bf16(bp[j]);
    float s0 = sigmoidf_(x.x), s1 = sigmoidf_(x.y);
    p1[j] = pack_bf16(dgv.x * y.x * s0 * (1.f + x.x * (1.f - s0)), dgv.y * y.y * s1 * (1.f + x.y * (1.f - s1)));
    p3[j] = pack_bf16(dgv.x * x.x * s0, dgv.y * x.y * s1);
  }
  reinterpret_cast<uint4*>(dh1)[i] = o1;
  reinterpret_cast<uint4*>(dh3)[i] = o3;
}

// ---- cross-entropy slab: one block per row ------------------------------------------------------------------------
// row_loss[r] = (lse - logit[target]) * valid * inv_n ; dlogits = (softmax - onehot) * valid * inv_n
__global__ void ce_kernel(const bf16* __restrict__ logits, const long long* __restrict__ targets,
                          const float* __restrict__ inv_n_p, float* __restrict__ row_loss,
                          bf16* __restrict__ dlogits, int V) {
  __shared__ float sred[32];
  __shared__ float sb[2];
  const int row = blockIdx.x, tid = threadIdx.x, nw = blockDim.x >> 5;
  const bf16* lr = logits + (long long)row * V;
  float m = -INFINITY;
  for (int c = tid; c < V; c += blockDim.x) m = fmaxf(m, __bfloat162float(lr[c]));
  m = warp_max(m);
  if ((tid & 31) == 0) sred[tid >> 5] = m;
  __syncthreads();
  if (tid < 32) {
    float v = tid < nw ? sred[tid] : -INFINITY;
    v = warp_max(v);
    if (tid == 0) sb[0] = v;
  }
  __syncthreads();
  m = sb[0];
  float z = 0.f;
  for (int c = tid; c < V; c += blockDim.x) z += __expf(__bfloat162float(lr[c]) - m);
  z = warp_sum(z);
  __syncthreads();
  if ((tid & 31) == 0) sred[tid >> 5] = z;
  __syncthreads();
  if (tid < 32) {
    float v = tid < nw ? sred[tid] : 0.f;
    v = warp_sum(v);
    if (tid == 0) sb[1] = v;
  }
  __syncthreads();
  z = sb[1];
  const long long tg = targets[row];
  const bool valid = tg >= 0;
  const float inv_n = *inv_n_p, lse = m + __logf(z);
  if (tid == 0) row_loss[row] = valid ? (lse - __bfloat162float(lr[tg])) * inv_n : 0.f;
  if (dlogits) {
    bf16* dr = dlogits + (long long)row * V;
    const float sc = valid ? inv_n : 0.f, rz = 1.f / z;
    for (int c = tid; c < V; c += blockDim.x) {
      float p = __expf(__bfloat162float(lr[c]) - m) * rz;
      if (c == tg) p -= 1.f;
      dr[c] = __float2bfloat16(p * sc);
    }
  }
}

// ---- embedding backward, run-to-run deterministic ----------------------------------------------
// tok_sorted: the batch's token ids in ascending order, order[p]: the flat position whose id is
// tok_sorted[p] (a stable sort, so equal ids keep position order).  The block at the first slot of a
// run of equal ids adds that run's rows of dx, in position order, into the id's row of the fp32
// table gradient; every other block exits.  No atomics: each table row has exactly one writer and a
// fixed summation order.  One thread per 4 columns.
template <typename TD>
__global__ void embed_bwd_sorted_kernel(const long long* __restrict__ tok_sorted,
                                        const long long* __restrict__ order, const TD* __restrict__ dx,
                                        float* __restrict__ gw, int n, int d) {
  const int p = blockIdx.x;
  const long long tok = tok_sorted[p];
  if (p > 0 && tok_sorted[p - 1] == tok) return;
  for (int c = threadIdx.x * 4; c < d; c += blockDim.x * 4) {
    float4 acc = *reinterpret_cast<const float4*>(gw + tok * d + c);
    for (int q = p; q < n && tok_sorted[q] == tok; ++q) {
      const TD* r = dx + order[q] * d + c;
      if constexpr (sizeof(TD) == 2) {
        uint2 u = *reinterpret_cast<const uint2*>(r);
        float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y);
        acc.x += a.x; acc.y += a.y; acc.z += b.x; acc.w += b.y;
      } else {
        float4 v = *reinterpret_cast<const float4*>(r);
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
      }
    }
    *reinterpret_cast<float4*>(gw + tok * d + c) = acc;
  }
}

}  // namespace

extern "C" {

int dmb_rms_fwd(const void* x, long long xs, const void* w, void* y, float* rstd, int rows, int d,
                float eps, cudaStream_t st) {
  if (d % 8) return -1;
  rms_fwd_kernel<<<(rows + 7) / 8, 256, 0, st>>>((const bf16*)x, xs, (const bf16*)w, (bf16*)y, rstd, rows,
                                                 d, eps);
  DMB_CHECK_LAUNCH();
  return 0;
}

// dy_f32 / out_f32: element types of dy and of residual/out
int dmb_rms_bwd_dx(const void* dy, int dy_f32, const void* x, long long xs, const void* w,
                   const float* rstd, const void* residual, void* out, int out_f32, int rows, int d,
                   cudaStream_t st) {
  dim3 grid((rows + 7) / 8), blk(256);
  if (dy_f32 && out_f32)
    rms_bwd_dx_kernel<float, float><<<grid, blk, 0, st>>>((const float*)dy, (const bf16*)x, xs, (const bf16*)w, rstd, (const float*)residual, (float*)out, rows, d);
  else if (dy_f32)
    rms_bwd_dx_kernel<float, bf16><<<grid, blk, 0, st>>>((const float*)dy, (const bf16*)x, xs, (const bf16*)w, rstd, (const bf16*)residual, (bf16*)out, rows, d);
  else if (out_f32)
    rms_bwd_dx_kernel<bf16, float><<<grid, blk, 0, st>>>((const bf16*)dy, (const bf16*)x, xs, (const bf16*)w, rstd, (const float*)residual, (float*)out, rows, d);
  else
    rms_bwd_dx_kernel<bf16, bf16><<<grid, blk, 0, st>>>((const bf16*)dy, (const bf16*)x, xs, (const bf16*)w, rstd, (const bf16*)residual, (bf16*)out, rows, d);
  DMB_CHECK_LAUNCH();
  return 0;
}

// out[col] += sum_rows dy * (x * rstd)   (x == nullptr: plain column sum).  `partial` is caller
// scratch of nsplit * d floats.
int dmb_col_reduce_acc(const void* dy, int dy_f32, const void* x, long long xs, const float* rstd,
                       float* partial, int nsplit, float* out, int rows, int d, cudaStream_t st) {
  int rps = (rows + nsplit - 1) / nsplit;
  dim3 grid((d + 63) / 64, nsplit), blk(512);
  if (dy_f32)
    col_partial_kernel<float><<<grid, blk, 0, st>>>((const float*)dy, (const bf16*)x, xs, x ? rstd : nullptr, partial, rows, d, rps);
  else
    col_partial_kernel<bf16><<<grid, blk, 0, st>>>((const bf16*)dy, (const bf16*)x, xs, x ? rstd : nullptr, partial, rows, d, rps);
  DMB_CHECK_LAUNCH();
  reduce_partials_kernel<<<(d + 255) / 256, 256, 0, st>>>(partial, out, nsplit, d);
  DMB_CHECK_LAUNCH();
  return 0;
}

// ---- column reduction for callers that cannot allocate ---------------------------------------
// See noalloc.h.  The partial sums live in a fixed array inside this library instead of caller
// memory.  Every entry the second kernel reads is written by the first one in the same call, so
// nothing in the array has to start at zero and the previous call's contents do not matter.
static __device__ __align__(256) float g_noalloc_partials[DMB_NOALLOC_MAX_SPLIT * DMB_NOALLOC_MAX_COLS];
// per-device address cache: two host threads that race through the first call on a device both
// store the same address, so the slot needs no lock
static float* g_noalloc_ptr[DMB_NOALLOC_MAX_DEVICES] = {nullptr};
static thread_local char g_noalloc_err[256] = "";   // one message buffer per calling host thread

const char* dmb_noalloc_last_error() { return g_noalloc_err; }

int dmb_col_reduce_acc_noalloc(const void* dy, int dy_f32, const void* x, long long xs, const float* rstd,
                               float* out, int rows, int d, cudaStream_t st) {
  g_noalloc_err[0] = 0;
  if (d <= 0 || rows <= 0 || d > DMB_NOALLOC_MAX_COLS) {
    snprintf(g_noalloc_err, sizeof(g_noalloc_err),
             "dmb_col_reduce_acc_noalloc: %d columns / %d rows not supported (1 <= columns <= %d, rows >= 1); "
             "use dmb_col_reduce_acc with caller scratch for wider inputs", d, rows, DMB_NOALLOC_MAX_COLS);
    return DMB_NOALLOC_E_SIZE;
  }
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= DMB_NOALLOC_MAX_DEVICES) {
    snprintf(g_noalloc_err, sizeof(g_noalloc_err), "dmb_col_reduce_acc_noalloc: no usable current device (%d, CUDA error %d)", dev, (int)e);
    return DMB_NOALLOC_E_DEVICE;
  }
  if (g_noalloc_ptr[dev] == nullptr) {
    // one-time set-up for this device: in host code the array's name is only a handle, the device
    // address has to be asked for while that device is current
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_noalloc_partials);
    if (e != cudaSuccess || p == nullptr) {
      snprintf(g_noalloc_err, sizeof(g_noalloc_err), "dmb_col_reduce_acc_noalloc: cudaGetSymbolAddress failed on device %d (CUDA error %d)", dev, (int)e);
      return DMB_NOALLOC_E_DEVICE;
    }
    g_noalloc_ptr[dev] = p;
  }
  int nsplit = rows / 64;
  if (nsplit < 1) nsplit = 1;
  if (nsplit > DMB_NOALLOC_MAX_SPLIT) nsplit = DMB_NOALLOC_MAX_SPLIT;
  return dmb_col_reduce_acc(dy, dy_f32, x, xs, rstd, g_noalloc_ptr[dev], nsplit, out, rows, d, st);
}

int dmb_rope(const void* x, int in_f32, long long bs, long long rs, const float* cosb, const float* sinb,
             void* out, int out_f32, int B, int T, int H, int DH, float sign, cudaStream_t st) {
  long long total = (long long)B * T * H * (DH / 2);
  dim3 grid((unsigned)((total + 255) / 256)), blk(256);
  if (in_f32 && out_f32)
    rope_kernel<float, float><<<grid, blk, 0, st>>>((const float*)x, bs, rs, cosb, sinb, (float*)out, B, T, H, DH, sign);
  else if (in_f32)
    rope_kernel<float, bf16><<<grid, blk, 0, st>>>((const float*)x, bs, rs, cosb, sinb, (bf16*)out, B, T, H, DH, sign);
  else if (out_f32)
    rope_kernel<bf16, float><<<grid, blk, 0, st>>>((const bf16*)x, bs, rs, cosb, sinb, (float*)out, B, T, H, DH, sign);
  else
    rope_kernel<bf16, bf16><<<grid, blk, 0, st>>>((const bf16*)x, bs, rs, cosb, sinb, (bf16*)out, B, T, H, DH, sign);
  DMB_CHECK_LAUNCH();
  return 0;
}

int dmb_swiglu_fwd(const void* h1, const void* h3, void* g, long long n, cudaStream_t st) {
  if (n % 8) return -1;
  long long n8 = n / 8;
  swiglu_fwd_kernel<<<(unsigned)((n8 + 255) / 256), 256, 0, st>>>((const bf16*)h1, (const bf16*)h3, (bf16*)g, n8);
  DMB_CHECK_LAUNCH();
  return 0;
}

int dmb_swiglu_bwd(const void* dg, const void* h1, const void* h3, void* dh1, void* dh3, long long n,
                   cudaStream_t st) {
  if (n % 8) return -1;
  long long n8 = n / 8;
  swiglu_bwd_kernel<<<(unsigned)((n8 + 255) / 256), 256, 0, st>>>((const bf16*)dg, (const bf16*)h1, (const bf16*)h3, (bf16*)dh1, (bf16*)dh3, n8);
  DMB_CHECK_LAUNCH();
  return 0;
}

int dmb_ce(const void* logits, const long long* targets, const float* inv_n, float* row_loss,
           void* dlogits, int rows, int V, cudaStream_t st) {
  ce_kernel<<<rows, 512, 0, st>>>((const bf16*)logits, targets, inv_n, row_loss, (bf16*)dlogits, V);
  DMB_CHECK_LAUNCH();
  return 0;
}

// gw[tok] += sum of dx rows whose token id is tok, in position order (see the kernel's comment)
int dmb_embed_bwd_sorted(const long long* tok_sorted, const long long* order, const void* dx, int dx_f32,
                         float* gw, int n, int d, cudaStream_t st) {
  if (d % 4 || n <= 0) return -1;
  int threads = d / 4 < 256 ? ((d / 4 + 31) / 32) * 32 : 256;
  if (dx_f32)
    embed_bwd_sorted_kernel<float><<<n, threads, 0, st>>>(tok_sorted, order, (const float*)dx, gw, n, d);
  else
    embed_bwd_sorted_kernel<bf16><<<n, threads, 0, st>>>(tok_sorted, order, (const bf16*)dx, gw, n, d);
  DMB_CHECK_LAUNCH();
  return 0;
}

}  // extern "C"
