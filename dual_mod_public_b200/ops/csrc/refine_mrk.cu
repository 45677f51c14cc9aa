// Write law of the mult_res family (the reference's 1.3B recipe), forward and backward.
//
// Per row, with rstd = 1/rms(o) from the per-head sums of squares and cg = rstd * raw, raw = o @ W'^T,
// W' = [W_kctx ; V_map ; W_gk_u ; W_gv_u] * w_ctx (context-norm gain folded into the columns):
//   cg   = [k_c | v_m | gate-u logits k | gate-u logits v]
//   v_in = lam * (rstd o w_ctx) + sigmoid(vgx) * tanh(v_m)            vgx = x-logits of the branch gate (+ bias)
//   v_c  = v_in @ W_vctx^T                                            (a GEMM between the two kernels)
//   k_n  = per-head rms(k_c) * k_gain[h]                              (eps 1e-6)
//   k''  = g_k k + (1 - g_k) k_n,  v'' = g_v v + (1 - g_v) v_c        g = sigmoid(glx + gate-u logits), fp32
//   v''  : the first pin_cols columns keep the raw value; every head is projected onto the L2 ball of radius tau
//   K    = RoPE(k'')
// Thread map as in refine.cu (refine_common.cuh): one thread owns 8 rotation pairs of one head, the DH/16
// threads of a head are adjacent lanes, per-head sums go through `head_sum`.  All lanes stay alive to the
// end (loads are clamped to the last valid element, stores predicated) so the shuffles are well defined.
#include "refine_common.cuh"

namespace {

__device__ __forceinline__ float tanhf_(float x) {
  const float e = __expf(-2.f * fabsf(x));
  const float t = (1.f - e) / (1.f + e);
  return x < 0.f ? -t : t;
}

struct Loc {
  Where w;
  bool ok;
  int per_head, h;
};
__device__ __forceinline__ Loc locate_all(int B, int C, int H, int DH) {
  Loc L;
  const int half = DH >> 1;
  L.per_head = half >> 3;
  const long long total = (long long)B * C * H * L.per_head;
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  L.ok = i < total;
  if (!L.ok) i = total - 1;
  locate(L.w, i, B, C, H, DH);
  L.h = L.w.c0 / DH;
  return L;
}

// ---- v_in ----------------------------------------------------------------------------------------
__global__ void mrk_vin_fwd_kernel(const bf16* __restrict__ raw, const float* __restrict__ ssq, const bf16* __restrict__ o,
                                   const bf16* __restrict__ w_ctx, const bf16* __restrict__ vgx, TView vx,
                                   bf16* __restrict__ vin, int B, int C, int H, int DH, float lam, float eps) {
  const Loc L = locate_all(B, C, H, DH);
  const Where& w = L.w;
  const int d = H * DH;
  const float rs = row_rstd(ssq + w.row * H, H, d, eps);
  const bf16* rr = raw + w.row * 4 * d + d;                 // the v_m block
  const bf16* xr = vgx + w.b * vx.bs + w.t * vx.rs;
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    const int col = e ? w.c1 : w.c0;
    const V8 vm = ld8(rr + col), ov = ld8(o + w.row * d + col), wc = ld8(w_ctx + col), gx = ld8(xr + col);
    V8 r;
#pragma unroll
    for (int i = 0; i < 8; ++i)
      r.x[i] = lam * ov.x[i] * rs * wc.x[i] + sigmoidf_(gx.x[i]) * tanhf_(vm.x[i] * rs);
    if (L.ok) st8(vin + w.row * d + col, r);
  }
}

// dvin [rows, d] -> dcg's v_m block, the gate x-logits' gradient (+=), the direct path's d uhat (fp32)
__global__ void mrk_vin_bwd_kernel(const bf16* __restrict__ dvin, const bf16* __restrict__ raw, const float* __restrict__ ssq,
                                   const bf16* __restrict__ w_ctx, const bf16* __restrict__ vgx, TView vx,
                                   bf16* __restrict__ dcg, float* __restrict__ dvgx_acc, TView vdx,
                                   float* __restrict__ du_hat, int B, int C, int H, int DH, float lam, float eps) {
  const Loc L = locate_all(B, C, H, DH);
  const Where& w = L.w;
  const int d = H * DH;
  const float rs = row_rstd(ssq + w.row * H, H, d, eps);
  const bf16* rr = raw + w.row * 4 * d + d;
  const bf16* xr = vgx + w.b * vx.bs + w.t * vx.rs;
  float* dxr = dvgx_acc + w.b * vdx.bs + w.t * vdx.rs;
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    const int col = e ? w.c1 : w.c0;
    const V8 g = ld8(dvin + w.row * d + col), vm = ld8(rr + col), wc = ld8(w_ctx + col), gx = ld8(xr + col);
    V8 dvm, dgx, duh;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float t = tanhf_(vm.x[i] * rs), sg = sigmoidf_(gx.x[i]);
      dvm.x[i] = g.x[i] * sg * (1.f - t * t);
      dgx.x[i] = g.x[i] * t * sg * (1.f - sg);
      duh.x[i] = lam * g.x[i] * wc.x[i];
    }
    if (L.ok) {
      st8(dcg + w.row * 4 * d + d + col, dvm);
      acc8f(dxr + col, dgx);
      st8f(du_hat + w.row * d + col, duh);
    }
  }
}

// ---- blend / norm / clamp / rope -------------------------------------------------------------------
struct Fwd {
  V8 kc[2], gk[2], gv[2], vpre[2], kraw[2], vdiff[2];      // kc: rstd-scaled ctx key; vdiff = v_raw - v_c
  float rs, rh, gain, nrm2, shrink;                        // normalised ctx key k_n = kc * rh * gain
};
// everything the forward computes for this thread's 16 elements (shared by forward and backward)
__device__ __forceinline__ void mrk_forward_parts(Fwd& f, const Loc& L, const bf16* raw, const bf16* vc, const float* ssq,
                                                  const bf16* gr, const bf16* kr, const bf16* vr, const float* k_gain,
                                                  int H, int DH, int pin_cols, float tau, float eps) {
  const Where& w = L.w;
  const int d = H * DH;
  f.rs = row_rstd(ssq + w.row * H, H, d, eps);
  const bf16* rr = raw + w.row * 4 * d;
  float s2 = 0.f;
  V8 vraw[2], vcv[2];
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    const int col = e ? w.c1 : w.c0;
    f.kc[e] = ld8(rr + col);
    const V8 gku = ld8(rr + 2 * d + col), gvu = ld8(rr + 3 * d + col), gxk = ld8(gr + col), gxv = ld8(gr + d + col);
    f.kraw[e] = ld8(kr + col);
    vraw[e] = ld8(vr + col);
    vcv[e] = ld8(vc + w.row * d + col);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      f.kc[e].x[i] *= f.rs;
      s2 += f.kc[e].x[i] * f.kc[e].x[i];
      f.gk[e].x[i] = sigmoidf_(gxk.x[i] + f.rs * gku.x[i]);
      f.gv[e].x[i] = sigmoidf_(gxv.x[i] + f.rs * gvu.x[i]);
    }
  }
  f.rh = rsqrtf(head_sum(s2, L.per_head) / DH + 1e-6f);
  f.gain = k_gain[L.h];
  float n2 = 0.f;
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    const int col = e ? w.c1 : w.c0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float gv = f.gv[e].x[i];
      f.vdiff[e].x[i] = vraw[e].x[i] - vcv[e].x[i];
      f.vpre[e].x[i] = (col + i < pin_cols) ? vraw[e].x[i] : vcv[e].x[i] + gv * f.vdiff[e].x[i];
      n2 += f.vpre[e].x[i] * f.vpre[e].x[i];
    }
  }
  f.nrm2 = fmaxf(head_sum(n2, L.per_head), 1e-40f);
  f.shrink = (tau > 0.f) ? fminf(1.f, tau * rsqrtf(f.nrm2)) : 1.f;
}

__global__ void mrk_refine_fwd_kernel(const bf16* __restrict__ raw, const bf16* __restrict__ vc, const float* __restrict__ ssq,
                                      const bf16* __restrict__ glx, TView vg, const bf16* __restrict__ k, TView vk,
                                      const bf16* __restrict__ v, TView vv, const float* __restrict__ cosb,
                                      const float* __restrict__ sinb, const float* __restrict__ k_gain,
                                      bf16* __restrict__ Kout, bf16* __restrict__ Vout, TView vo_, int B, int C, int H,
                                      int DH, int pin_cols, float tau, float eps) {
  const Loc L = locate_all(B, C, H, DH);
  const Where& w = L.w;
  const int half = DH >> 1;
  Fwd f;
  mrk_forward_parts(f, L, raw, vc, ssq, glx + w.b * vg.bs + w.t * vg.rs, k + w.b * vk.bs + w.t * vk.rs,
                    v + w.b * vv.bs + w.t * vv.rs, k_gain, H, DH, pin_cols, tau, eps);
  const V8 cs = ld8f(cosb + w.t * half + w.p0), sn = ld8f(sinb + w.t * half + w.p0);
  V8 kk[2], vo[2];
#pragma unroll
  for (int e = 0; e < 2; ++e)
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float gk = f.gk[e].x[i];
      kk[e].x[i] = gk * f.kraw[e].x[i] + (1.f - gk) * (f.kc[e].x[i] * f.rh * f.gain);
      vo[e].x[i] = f.vpre[e].x[i] * f.shrink;
    }
  V8 k0, k1;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    k0.x[i] = kk[0].x[i] * cs.x[i] - kk[1].x[i] * sn.x[i];
    k1.x[i] = kk[1].x[i] * cs.x[i] + kk[0].x[i] * sn.x[i];
  }
  if (L.ok) {
    const long long o = w.b * vo_.bs + w.t * vo_.rs;
    st8(Kout + o + w.c0, k0);
    st8(Kout + o + w.c1, k1);
    st8(Vout + o + w.c0, vo[0]);
    st8(Vout + o + w.c1, vo[1]);
  }
}

// dK / dV fp32 dense [B,C,H,DH].  Writes dcg blocks 0, 2, 3 (bf16 [rows,4d]; block 1 = d v_m comes from
// mrk_vin_bwd), uhat = o * rstd, dvc (bf16 [rows,d]) and the per-(row, head) k_gain gradient dkg [rows,H];
// accumulates dk_acc / dv_acc [.., d] and dglx_acc [.., 2d] (fp32, +=).
template <int MINB>
__global__ void __launch_bounds__(128, MINB) mrk_refine_bwd_kernel(const float* __restrict__ dK, const float* __restrict__ dV, TView vdo,
                                      const bf16* __restrict__ raw,
                                      const bf16* __restrict__ vc, const float* __restrict__ ssq, const bf16* __restrict__ o,
                                      const bf16* __restrict__ glx, TView vg, const bf16* __restrict__ k, TView vk,
                                      const bf16* __restrict__ v, TView vv, const float* __restrict__ cosb,
                                      const float* __restrict__ sinb, const float* __restrict__ k_gain,
                                      bf16* __restrict__ dcg, bf16* __restrict__ uhat, bf16* __restrict__ dvc,
                                      float* __restrict__ dkg, float* __restrict__ dk_acc, TView vdk,
                                      float* __restrict__ dv_acc, TView vdv, float* __restrict__ dglx_acc, TView vdg, int B,
                                      int C, int H, int DH, int pin_cols, float tau, float eps) {
  const Loc L = locate_all(B, C, H, DH);
  const Where& w = L.w;
  const int d = H * DH, half = DH >> 1;
  Fwd f;
  mrk_forward_parts(f, L, raw, vc, ssq, glx + w.b * vg.bs + w.t * vg.rs, k + w.b * vk.bs + w.t * vk.rs,
                    v + w.b * vv.bs + w.t * vv.rs, k_gain, H, DH, pin_cols, tau, eps);
  const V8 cs = ld8f(cosb + w.t * half + w.p0), sn = ld8f(sinb + w.t * half + w.p0);
  const long long ob = w.row * d;
  const long long gb = w.b * vdo.bs + w.t * vdo.rs;       // dK / dV may be a window of a longer [B, T, d] array
  const V8 a = ld8f(dK + gb + w.c0), bq = ld8f(dK + gb + w.c1);
  V8 dkpp[2], dvo[2] = {ld8f(dV + gb + w.c0), ld8f(dV + gb + w.c1)};
#pragma unroll
  for (int i = 0; i < 8; ++i) {            // transpose of the rotation
    dkpp[0].x[i] = a.x[i] * cs.x[i] + bq.x[i] * sn.x[i];
    dkpp[1].x[i] = bq.x[i] * cs.x[i] - a.x[i] * sn.x[i];
  }
  // projection onto the ball: inside -> identity; outside -> shrink * (dv - vpre (dv . vpre) / |vpre|^2)
  float dot = 0.f;
#pragma unroll
  for (int e = 0; e < 2; ++e)
#pragma unroll
    for (int i = 0; i < 8; ++i) dot += dvo[e].x[i] * f.vpre[e].x[i];
  dot = head_sum(dot, L.per_head);
  const bool outside = f.shrink < 1.f;
  const float proj = dot / f.nrm2;
  const float gain = f.gain;
  float s_g = 0.f;
#pragma unroll
  for (int e = 0; e < 2; ++e)
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (outside) dvo[e].x[i] = f.shrink * (dvo[e].x[i] - f.vpre[e].x[i] * proj);
      const float dkn = dkpp[e].x[i] * (1.f - f.gk[e].x[i]);
      s_g += dkn * (f.kc[e].x[i] * f.rh);              // d k_n . normalised ctx key
    }
  s_g = head_sum(s_g, L.per_head);
  const float s_dx = s_g * gain / DH;
  bf16* dr = dcg + w.row * 4 * d;
  float* dkr = dk_acc + w.b * vdk.bs + w.t * vdk.rs;
  float* dvr = dv_acc + w.b * vdv.bs + w.t * vdv.rs;
  float* dgr = dglx_acc + w.b * vdg.bs + w.t * vdg.rs;
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    const int col = e ? w.c1 : w.c0;
    const V8 ov = ld8(o + ob + col);
    V8 dkc, dgk, dgv, dvcv, dkk, dvv, uh;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float gk = f.gk[e].x[i], gv = f.gv[e].x[i];
      const bool pinned = col + i < pin_cols;
      const float dvp = pinned ? 0.f : dvo[e].x[i];
      const float xh = f.kc[e].x[i] * f.rh;
      dkc.x[i] = f.rh * (dkpp[e].x[i] * (1.f - gk) * gain - xh * s_dx);
      dgk.x[i] = dkpp[e].x[i] * (f.kraw[e].x[i] - xh * gain) * gk * (1.f - gk);
      dgv.x[i] = dvp * f.vdiff[e].x[i] * gv * (1.f - gv);
      dvcv.x[i] = dvp * (1.f - gv);
      dkk.x[i] = dkpp[e].x[i] * gk;
      dvv.x[i] = pinned ? dvo[e].x[i] : dvp * gv;
      uh.x[i] = ov.x[i] * f.rs;
    }
    if (L.ok) {
      st8(dr + col, dkc);
      st8(dr + 2 * d + col, dgk);
      st8(dr + 3 * d + col, dgv);
      st8(dvc + ob + col, dvcv);
      st8(uhat + ob + col, uh);
      acc8f(dkr + col, dkk);
      acc8f(dvr + col, dvv);
      if (dglx_acc) {
        acc8f(dgr + col, dgk);
        acc8f(dgr + d + col, dgv);
      }
    }
  }
  if (L.ok && (threadIdx.x % L.per_head) == 0) dkg[w.row * H + L.h] = s_g;
}

}  // namespace

namespace { int g_mrk_bwd_minb = 4; }

extern "C" {

static inline unsigned mrk_blocks(int B, int C, int H, int DH, int threads) {
  const long long total = (long long)B * C * H * (DH / 16);
  return (unsigned)((total + threads - 1) / threads);
}

int dmb_mrk_vin_fwd(const void* raw, const float* ssq, const void* o, const void* w_ctx, const void* vgx, TView vx,
                    void* vin, int B, int C, int H, int DH, float lam, float eps, cudaStream_t st) {
  if (DH % 16) return -1;
  mrk_vin_fwd_kernel<<<mrk_blocks(B, C, H, DH, 256), 256, 0, st>>>((const bf16*)raw, ssq, (const bf16*)o, (const bf16*)w_ctx,
                                                                 (const bf16*)vgx, vx, (bf16*)vin, B, C, H, DH, lam, eps);
  DMB_CHECK_LAUNCH();
  return 0;
}

int dmb_mrk_vin_bwd(const void* dvin, const void* raw, const float* ssq, const void* w_ctx, const void* vgx, TView vx,
                    void* dcg, float* dvgx_acc, TView vdx, float* du_hat, int B, int C, int H, int DH, float lam, float eps,
                    cudaStream_t st) {
  if (DH % 16) return -1;
  mrk_vin_bwd_kernel<<<mrk_blocks(B, C, H, DH, 256), 256, 0, st>>>((const bf16*)dvin, (const bf16*)raw, ssq, (const bf16*)w_ctx,
                                                                 (const bf16*)vgx, vx, (bf16*)dcg, dvgx_acc, vdx, du_hat, B, C,
                                                                 H, DH, lam, eps);
  DMB_CHECK_LAUNCH();
  return 0;
}

int dmb_mrk_refine_fwd(const void* raw, const void* vc, const float* ssq, const void* glx, TView vg, const void* k, TView vk,
                       const void* v, TView vv, const float* cosb, const float* sinb, const float* k_gain, void* Kout,
                       void* Vout, TView vo, int B, int C, int H, int DH, int pin_cols, float tau, float eps, cudaStream_t st) {
  if (DH % 16) return -1;
  mrk_refine_fwd_kernel<<<mrk_blocks(B, C, H, DH, 128), 128, 0, st>>>(
      (const bf16*)raw, (const bf16*)vc, ssq, (const bf16*)glx, vg, (const bf16*)k, vk, (const bf16*)v, vv, cosb, sinb, k_gain,
      (bf16*)Kout, (bf16*)Vout, vo, B, C, H, DH, pin_cols, tau, eps);
  DMB_CHECK_LAUNCH();
  return 0;
}

// resident blocks per SM the compiler sizes the backward kernel's registers for (2, 3 or 4; measured at 8192 rows x
// 2304: 274 / 226 / 216 us, the last with 128 registers and 180 bytes of spills)
void dmb_mrk_refine_bwd_minblocks(int n) { g_mrk_bwd_minb = n; }

int dmb_mrk_refine_bwd(const float* dK, const float* dV, TView vdo, const void* raw, const void* vc, const float* ssq, const void* o,
                       const void* glx, TView vg, const void* k, TView vk, const void* v, TView vv, const float* cosb,
                       const float* sinb, const float* k_gain, void* dcg, void* uhat, void* dvc, float* dkg, float* dk_acc,
                       TView vdk, float* dv_acc, TView vdv, float* dglx_acc, TView vdg, int B, int C, int H, int DH,
                       int pin_cols, float tau, float eps, cudaStream_t st) {
  if (DH % 16) return -1;
#define RB_GO(MB) mrk_refine_bwd_kernel<MB><<<mrk_blocks(B, C, H, DH, 128), 128, 0, st>>>( \
      dK, dV, vdo, (const bf16*)raw, (const bf16*)vc, ssq, (const bf16*)o, (const bf16*)glx, vg, (const bf16*)k, vk, (const bf16*)v, \
      vv, cosb, sinb, k_gain, (bf16*)dcg, (bf16*)uhat, (bf16*)dvc, dkg, dk_acc, vdk, dv_acc, vdv, dglx_acc, vdg, B, C, H, DH, \
      pin_cols, tau, eps)
  if (g_mrk_bwd_minb == 2) { RB_GO(2); } else if (g_mrk_bwd_minb == 3) { RB_GO(3); } else { RB_GO(4); }
#undef RB_GO
  DMB_CHECK_LAUNCH();
  return 0;
}

}  // extern "C"
