// The Dual-Mod write law, forward and backward, fused into one pass over a chunk's rows.
//
// Inputs per row: raw[4d] = o @ W'^T (W' = packed ctx/gate weights with the context-norm gain
// folded into their columns, o the UN-normalised read), ssq[H] = per-head sums of squares of o
// (so rstd = rsqrt(sum(ssq)/d + eps) needs no pass over o), glx[2d] = x-half of the gate logits
// + bias, raw key k[d] and value v[d].  With cg = rstd * raw = [k_ctx | v_ctx | gk_u | gv_u]:
//   g = sigmoid(glx + g_u);  k'' = g_k k + (1-g_k) k_ctx;  v'' = g_v v + (1-g_v) v_ctx
//   K_out = RoPE(k'') (rotated once, at write), V_out = v'' (first pin_cols columns keep raw v).
// One thread owns 8 adjacent rotation pairs of one head: columns [c0, c0+8) and [c0+half, ..+8),
// so every access is a 16-byte vector.
#include "refine_common.cuh"

namespace {

__global__ void refine_fwd_kernel(const bf16* __restrict__ raw, const float* __restrict__ ssq,
                                  const bf16* __restrict__ glx, TView vg, const bf16* __restrict__ k, TView vk,
                                  const bf16* __restrict__ v, TView vv, const float* __restrict__ cosb,
                                  const float* __restrict__ sinb, bf16* __restrict__ Kout,
                                  bf16* __restrict__ Vout, TView vo_, int B, int C, int H, int DH, int pin_cols,
                                  float eps) {
  Where w;
  if (!locate(w, (long long)blockIdx.x * blockDim.x + threadIdx.x, B, C, H, DH)) return;
  const int d = H * DH, half = DH >> 1;
  const float rs = row_rstd(ssq + w.row * H, H, d, eps);
  const bf16* rr = raw + w.row * 4 * d;
  const bf16* gr = glx + w.b * vg.bs + w.t * vg.rs;
  const bf16* kr = k + w.b * vk.bs + w.t * vk.rs;
  const bf16* vr = v + w.b * vv.bs + w.t * vv.rs;
  const V8 cs = ld8f(cosb + w.t * half + w.p0), sn = ld8f(sinb + w.t * half + w.p0);
  V8 kk[2], vo[2];
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    const int col = e ? w.c1 : w.c0;
    const V8 kc = ld8(rr + col), vc = ld8(rr + d + col), gku = ld8(rr + 2 * d + col), gvu = ld8(rr + 3 * d + col);
    const V8 gxk = ld8(gr + col), gxv = ld8(gr + d + col), kraw = ld8(kr + col), vraw = ld8(vr + col);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float gk = sigmoidf_(gxk.x[i] + rs * gku.x[i]), gv = sigmoidf_(gxv.x[i] + rs * gvu.x[i]);
      kk[e].x[i] = gk * kraw.x[i] + (1.f - gk) * rs * kc.x[i];
      vo[e].x[i] = (col + i < pin_cols) ? vraw.x[i] : gv * vraw.x[i] + (1.f - gv) * rs * vc.x[i];
    }
  }
  V8 k0, k1;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    k0.x[i] = kk[0].x[i] * cs.x[i] - kk[1].x[i] * sn.x[i];
    k1.x[i] = kk[1].x[i] * cs.x[i] + kk[0].x[i] * sn.x[i];
  }
  const long long o = w.b * vo_.bs + w.t * vo_.rs;      // outputs may be rows of the tape itself
  st8(Kout + o + w.c0, k0);
  st8(Kout + o + w.c1, k1);
  st8(Vout + o + w.c0, vo[0]);
  st8(Vout + o + w.c1, vo[1]);
}

// dK / dV fp32 dense [B,C,H,DH]; writes dcg (bf16 [rows,4d], gradient w.r.t. cg = rstd*raw) and
// uhat = o * rstd (bf16 [rows,d]); accumulates dk_acc / dv_acc [.., d] and dglx_acc [.., 2d] (fp32, +=).
template <int MINB>
__global__ void __launch_bounds__(128, MINB) refine_bwd_kernel(const float* __restrict__ dK, const float* __restrict__ dV, TView vdo,
                                  const bf16* __restrict__ raw, const float* __restrict__ ssq,
                                  const bf16* __restrict__ o, const bf16* __restrict__ glx, TView vg,
                                  const bf16* __restrict__ k, TView vk, const bf16* __restrict__ v, TView vv,
                                  const float* __restrict__ cosb, const float* __restrict__ sinb,
                                  bf16* __restrict__ dcg, bf16* __restrict__ uhat, float* __restrict__ dk_acc,
                                  TView vdk, float* __restrict__ dv_acc, TView vdv, float* __restrict__ dglx_acc,
                                  TView vdg, int B, int C, int H, int DH, int pin_cols, float eps) {
  Where w;
  if (!locate(w, (long long)blockIdx.x * blockDim.x + threadIdx.x, B, C, H, DH)) return;
  const int d = H * DH, half = DH >> 1;
  const float rs = row_rstd(ssq + w.row * H, H, d, eps);
  const bf16* rr = raw + w.row * 4 * d;
  bf16* dr = dcg + w.row * 4 * d;
  const bf16* gr = glx + w.b * vg.bs + w.t * vg.rs;
  const bf16* kr = k + w.b * vk.bs + w.t * vk.rs;
  const bf16* vr = v + w.b * vv.bs + w.t * vv.rs;
  float* dkr = dk_acc + w.b * vdk.bs + w.t * vdk.rs;
  float* dvr = dv_acc + w.b * vdv.bs + w.t * vdv.rs;
  float* dgr = dglx_acc + w.b * vdg.bs + w.t * vdg.rs;
  const V8 cs = ld8f(cosb + w.t * half + w.p0), sn = ld8f(sinb + w.t * half + w.p0);
  const long long ob = w.row * d;
  const long long gb = w.b * vdo.bs + w.t * vdo.rs;       // dK / dV may be a window of a longer [B, T, d] array
  const V8 a = ld8f(dK + gb + w.c0), bq = ld8f(dK + gb + w.c1);
  V8 dkpp[2], dvpp[2] = {ld8f(dV + gb + w.c0), ld8f(dV + gb + w.c1)};
#pragma unroll
  for (int i = 0; i < 8; ++i) {            // transpose of the rotation
    dkpp[0].x[i] = a.x[i] * cs.x[i] + bq.x[i] * sn.x[i];
    dkpp[1].x[i] = bq.x[i] * cs.x[i] - a.x[i] * sn.x[i];
  }
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    const int col = e ? w.c1 : w.c0;
    const V8 kc = ld8(rr + col), vc = ld8(rr + d + col), gku = ld8(rr + 2 * d + col), gvu = ld8(rr + 3 * d + col);
    const V8 gxk = ld8(gr + col), gxv = ld8(gr + d + col), kraw = ld8(kr + col), vraw = ld8(vr + col);
    const V8 ov = ld8(o + ob + col);
    V8 dkc, dvc, dgk, dgv, dkk, dvv, uh;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float gk = sigmoidf_(gxk.x[i] + rs * gku.x[i]), gv = sigmoidf_(gxv.x[i] + rs * gvu.x[i]);
      const bool pinned = col + i < pin_cols;
      const float dvp = pinned ? 0.f : dvpp[e].x[i];
      dgk.x[i] = dkpp[e].x[i] * (kraw.x[i] - rs * kc.x[i]) * gk * (1.f - gk);
      dgv.x[i] = dvp * (vraw.x[i] - rs * vc.x[i]) * gv * (1.f - gv);
      dkc.x[i] = dkpp[e].x[i] * (1.f - gk);
      dvc.x[i] = dvp * (1.f - gv);
      dkk.x[i] = dkpp[e].x[i] * gk;
      dvv.x[i] = pinned ? dvpp[e].x[i] : dvp * gv;
      uh.x[i] = ov.x[i] * rs;
    }
    st8(dr + col, dkc);
    st8(dr + d + col, dvc);
    st8(dr + 2 * d + col, dgk);
    st8(dr + 3 * d + col, dgv);
    st8(uhat + ob + col, uh);
    acc8f(dkr + col, dkk);
    acc8f(dvr + col, dvv);
    if (dglx_acc) {             // null: the caller sums the gate columns of the stashed dcg once per layer instead
      acc8f(dgr + col, dgk);
      acc8f(dgr + d + col, dgv);
    }
  }
}

// out[b, t, :] (bf16, 2d wide, dense) = sum over the K sweeps of the gate-logit columns [2d, 4d) of the stashed
// d(ctx / gate logits): the rows of sweep s of cell ci sit at ((ci * K + s) * B + b) * c + i.  The gradient of a
// gate's x-logit equals that of its u-logit, so it is not accumulated per sweep but read back once per layer.
__global__ void stash_gate_sum_kernel(const bf16* __restrict__ stash, bf16* __restrict__ out, int B, int T, int c,
                                      int K, int d) {
  const int per_row = (2 * d) >> 3;
  const long long total = (long long)B * T * per_row;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int col = (int)(i % per_row) << 3;
    const long long row = i / per_row;
    const int t = (int)(row % T), b = (int)(row / T);
    const int ci = t / c, ii = t - ci * c;
    V8 acc = {};
    for (int s = 0; s < K; ++s) {
      const long long sr = (((long long)ci * K + s) * B + b) * c + ii;
      const V8 v = ld8(stash + sr * 4 * d + 2 * d + col);
#pragma unroll
      for (int e = 0; e < 8; ++e) acc.x[e] += v.x[e];
    }
    st8(out + row * 2 * d + col, acc);
  }
}

// d o of uhat = o * rstd (no gain): out = residual + rstd * (du - uhat * mean(du * uhat)); warp per row
template <typename TOUT>
__global__ void rmsn_bwd_kernel(const bf16* __restrict__ du, const bf16* __restrict__ o,
                                const float* __restrict__ ssq, const TOUT* __restrict__ residual,
                                const float* __restrict__ extra, TOUT* __restrict__ out, int rows, int d, int H,
                                float eps) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= rows) return;
  const float rs = row_rstd(ssq + (long long)row * H, H, d, eps);
  const bf16* dur = du + (long long)row * d;
  const bf16* orow = o + (long long)row * d;
  float acc = 0.f;
  const float* er = extra ? extra + (long long)row * d : nullptr;     // optional fp32 term added to du
  for (int c = lane * 8; c < d; c += 256) {
    V8 g = ld8(dur + c);
    const V8 x = ld8(orow + c);
    if (er) { const V8 q = ld8f(er + c);
#pragma unroll
      for (int i = 0; i < 8; ++i) g.x[i] += q.x[i]; }
#pragma unroll
    for (int i = 0; i < 8; ++i) acc += g.x[i] * x.x[i];
  }
  const float mean = warp_sum(acc) * rs / d;     // mean(du * uhat)
  for (int c = lane * 8; c < d; c += 256) {
    V8 g = ld8(dur + c);
    const V8 x = ld8(orow + c);
    if (er) { const V8 q = ld8f(er + c);
#pragma unroll
      for (int i = 0; i < 8; ++i) g.x[i] += q.x[i]; }
    V8 r;
#pragma unroll
    for (int i = 0; i < 8; ++i) r.x[i] = rs * (g.x[i] - x.x[i] * rs * mean);
    const long long off = (long long)row * d + c;
    if constexpr (sizeof(TOUT) == 4) {
      if (residual) { V8 q = ld8f((const float*)residual + off);
#pragma unroll
        for (int i = 0; i < 8; ++i) r.x[i] += q.x[i]; }
      st8f((float*)out + off, r);
    } else {
      if (residual) { V8 q = ld8((const bf16*)residual + off);
#pragma unroll
        for (int i = 0; i < 8; ++i) r.x[i] += q.x[i]; }
      st8((bf16*)out + off, r);
    }
  }
}

}  // namespace

namespace { int g_refine_bwd_minb = 4, g_refine_fwd_threads = 128; }

extern "C" {

void dmb_refine_fwd_threads(int n) { g_refine_fwd_threads = n == 256 ? 256 : 128; }

int dmb_refine_fwd(const void* raw, const float* ssq, const void* glx, TView vg, const void* k, TView vk,
                   const void* v, TView vv, const float* cosb, const float* sinb, void* Kout, void* Vout, TView vo,
                   int B, int C, int H, int DH, int pin_cols, float eps, cudaStream_t st) {
  if (DH % 16) return -1;
  long long total = (long long)B * C * H * (DH / 16);
  const int nt = g_refine_fwd_threads;          // 128: the 2048-row launch of a sweep fits in one wave of blocks
  refine_fwd_kernel<<<(unsigned)((total + nt - 1) / nt), nt, 0, st>>>(
      (const bf16*)raw, ssq, (const bf16*)glx, vg, (const bf16*)k, vk, (const bf16*)v, vv, cosb, sinb,
      (bf16*)Kout, (bf16*)Vout, vo, B, C, H, DH, pin_cols, eps);
  DMB_CHECK_LAUNCH();
  return 0;
}

// resident blocks per SM the compiler sizes the backward kernel's registers for (3, 4 or 5; 4: 128 registers, no
// spills, 37.8 against 42.3 us at 2048 rows x 1024)
void dmb_refine_bwd_minblocks(int n) { g_refine_bwd_minb = n; }

int dmb_refine_bwd(const float* dK, const float* dV, TView vdo, const void* raw, const float* ssq, const void* o,
                   const void* glx, TView vg, const void* k, TView vk, const void* v, TView vv, const float* cosb,
                   const float* sinb, void* dcg, void* uhat, float* dk_acc, TView vdk, float* dv_acc, TView vdv,
                   float* dglx_acc, TView vdg, int B, int C, int H, int DH, int pin_cols, float eps,
                   cudaStream_t st) {
  if (DH % 16) return -1;
  long long total = (long long)B * C * H * (DH / 16);
#define RB_GO(MB) refine_bwd_kernel<MB><<<(unsigned)((total + 127) / 128), 128, 0, st>>>( \
      dK, dV, vdo, (const bf16*)raw, ssq, (const bf16*)o, (const bf16*)glx, vg, (const bf16*)k, vk, (const bf16*)v, vv, \
      cosb, sinb, (bf16*)dcg, (bf16*)uhat, dk_acc, vdk, dv_acc, vdv, dglx_acc, vdg, B, C, H, DH, pin_cols, eps)
  if (g_refine_bwd_minb == 3) { RB_GO(3); } else if (g_refine_bwd_minb == 5) { RB_GO(5); } else { RB_GO(4); }
#undef RB_GO
  DMB_CHECK_LAUNCH();
  return 0;
}

int dmb_stash_gate_sum(const void* stash, void* out, int B, int T, int c, int K, int d, cudaStream_t st) {
  if (d % 8 || T % c) return -1;
  stash_gate_sum_kernel<<<1184, 256, 0, st>>>((const bf16*)stash, (bf16*)out, B, T, c, K, d);
  DMB_CHECK_LAUNCH();
  return 0;
}

int dmb_rmsn_bwd(const void* du, const void* o, const float* ssq, const void* residual, const float* extra, void* out,
                 int out_f32, int rows, int d, int H, float eps, cudaStream_t st) {
  if (d % 8) return -1;
  dim3 grid((rows + 7) / 8), blk(256);
  if (out_f32)
    rmsn_bwd_kernel<float><<<grid, blk, 0, st>>>((const bf16*)du, (const bf16*)o, ssq, (const float*)residual, extra, (float*)out, rows, d, H, eps);
  else
    rmsn_bwd_kernel<bf16><<<grid, blk, 0, st>>>((const bf16*)du, (const bf16*)o, ssq, (const bf16*)residual, extra, (bf16*)out, rows, d, H, eps);
  DMB_CHECK_LAUNCH();
  return 0;
}

}  // extern "C"
