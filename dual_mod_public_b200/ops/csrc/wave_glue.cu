// Glue between the attention kernels: the far / near partial algebra of the wavefront engine (one kernel
// each way) and the cell-end bookkeeping of the reverse scan.
//
// A window chunk's committed-prefix read is the log-sum-exp merge of a FAR partial (rows committed before
// the chunk entered; computed once per chunk, stored by absolute position) and a NEAR partial (the K-1
// chunks just before it; recomputed every sweep):
//
//   lse_c = log(exp(lse_f) + exp(lse_n)),  w_f = exp(lse_f - lse_c),  w_n = exp(lse_n - lse_c)
//   o_c   = w_f o_f + w_n o_n
//
// merge_fwd forms (o_c, lse_c, w_f, w_n); split_bwd takes d(o_c), d(lse_c) and produces, per (row, head),
//   d o_f = w_f d o_c          d lse_f = w_f (d o_c . (o_f - o_c) + d lse_c)      (accumulated over sweeps)
//   d o_n = w_n d o_c          corr_n  = d o_n . o_n - w_n (d o_c . (o_n - o_c) + d lse_c)
// which is what the prefix backward kernels consume (d o, corr = d o . o - d lse, lse).
//
// Layout: window tensors are dense [B, R, H, DH] / [B, R, H] (R rows of the window); tensors stored by
// absolute position are slices of [B, T, H, DH] / [B, T, H] buffers starting at the window's first row,
// so only their batch stride differs (bs_vec, bs_sca elements).  One warp per (batch, row, head).
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "common.cuh"

namespace {

using bf16 = __nv_bfloat16;

// Every lane of a (batch, row, head) warp owns PER = DH / 32 CONTIGUOUS elements of the head's row, read and written
// as one 8- or 16-byte access (rows are DH floats: 256 / 512 bytes per warp instruction).
template <int PER> __device__ __forceinline__ void ldf(const float* p, float (&r)[PER]) {
  if constexpr (PER == 2) { const float2 v = *reinterpret_cast<const float2*>(p); r[0] = v.x; r[1] = v.y; }
  else { const float4 v = *reinterpret_cast<const float4*>(p); r[0] = v.x; r[1] = v.y; r[2] = v.z; r[3] = v.w; }
}
template <int PER> __device__ __forceinline__ void stf(float* p, const float (&r)[PER]) {
  if constexpr (PER == 2) *reinterpret_cast<float2*>(p) = make_float2(r[0], r[1]);
  else *reinterpret_cast<float4*>(p) = make_float4(r[0], r[1], r[2], r[3]);
}
template <int PER> __device__ __forceinline__ void ldb(const bf16* p, float (&r)[PER]) {
  if constexpr (PER == 2) { const float2 v = unpack_bf16(*reinterpret_cast<const uint32_t*>(p)); r[0] = v.x; r[1] = v.y; }
  else {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    const float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y);
    r[0] = a.x; r[1] = a.y; r[2] = b.x; r[3] = b.y;
  }
}
template <int PER> __device__ __forceinline__ void stb(bf16* p, const float (&r)[PER]) {
  if constexpr (PER == 2) *reinterpret_cast<uint32_t*>(p) = pack_bf16(r[0], r[1]);
  else *reinterpret_cast<uint2*>(p) = make_uint2(pack_bf16(r[0], r[1]), pack_bf16(r[2], r[3]));
}
template <int PER> __device__ __forceinline__ void stv(float* p, const float (&r)[PER]) { stf<PER>(p, r); }
template <int PER> __device__ __forceinline__ void stv(bf16* p, const float (&r)[PER]) { stb<PER>(p, r); }

template <int DH>
__global__ void __launch_bounds__(256) merge_fwd_kernel(
    const float* __restrict__ o_f, const float* __restrict__ lse_f, long long bs_vec, long long bs_sca,
    const float* __restrict__ o_n, const float* __restrict__ lse_n, float* __restrict__ o_c,
    float* __restrict__ lse_c, float* __restrict__ w_f, float* __restrict__ w_n, int B, int R, int H) {
  const long long wid = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (wid >= (long long)B * R * H) return;
  const int h = (int)(wid % H);
  const long long br = wid / H;
  const int r = (int)(br % R), b = (int)(br / R);
  const long long s_abs = (long long)b * bs_sca + (long long)r * H + h;
  const long long v_abs = (long long)b * bs_vec + ((long long)r * H + h) * DH;
  const float lf = lse_f[s_abs], ln = lse_n[wid];
  const float m = fmaxf(lf, ln);
  const float lc = m + __logf(__expf(lf - m) + __expf(ln - m));
  const float wf = __expf(lf - lc), wn = __expf(ln - lc);
  constexpr int PER = DH / 32;
  float f_[PER], n_[PER], c_[PER];
  ldf<PER>(o_f + v_abs + lane * PER, f_);
  ldf<PER>(o_n + wid * DH + lane * PER, n_);
#pragma unroll
  for (int e = 0; e < PER; ++e) c_[e] = wf * f_[e] + wn * n_[e];
  stf<PER>(o_c + wid * DH + lane * PER, c_);
  if (lane == 0) {
    lse_c[wid] = lc;
    w_f[wid] = wf;
    w_n[wid] = wn;
  }
}

template <int DH, typename TD>
__global__ void __launch_bounds__(256) split_bwd_kernel(
    const float* __restrict__ do_c, const float* __restrict__ dlse_c, const float* __restrict__ o_c,
    const float* __restrict__ o_n, const float* __restrict__ lse_n, const float* __restrict__ w_f,
    const float* __restrict__ w_n, const float* __restrict__ o_f, float* __restrict__ DOf,
    float* __restrict__ DLf, TD* __restrict__ docn, float* __restrict__ corrn, float* __restrict__ corrn_dense,
    float* __restrict__ lsen, long long bs_vec, long long bs_sca, int B, int R, int H) {
  const long long wid = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (wid >= (long long)B * R * H) return;
  const int h = (int)(wid % H);
  const long long br = wid / H;
  const int r = (int)(br % R), b = (int)(br / R);
  const long long s_abs = (long long)b * bs_sca + (long long)r * H + h;
  const long long v_abs = (long long)b * bs_vec + ((long long)r * H + h) * DH;
  const float wf = w_f[wid], wn = w_n[wid], dl = dlse_c[wid];
  constexpr int PER = DH / 32;
  float g[PER], on[PER], oc[PER], of[PER], acc[PER], dn[PER], dotf = 0.f, dotn = 0.f, donon = 0.f;
  ldf<PER>(do_c + wid * DH + lane * PER, g);
  ldf<PER>(o_n + wid * DH + lane * PER, on);
  ldf<PER>(o_c + wid * DH + lane * PER, oc);
  ldf<PER>(o_f + v_abs + lane * PER, of);
  ldf<PER>(DOf + v_abs + lane * PER, acc);
#pragma unroll
  for (int e = 0; e < PER; ++e) {
    dotf += g[e] * (of[e] - oc[e]);
    dotn += g[e] * (on[e] - oc[e]);
    donon += g[e] * on[e];
    acc[e] += wf * g[e];
    dn[e] = wn * g[e];
  }
  dotf = warp_sum(dotf);
  dotn = warp_sum(dotn);
  donon = warp_sum(donon);
  stf<PER>(DOf + v_abs + lane * PER, acc);
  stv<PER>(docn + v_abs + lane * PER, dn);
  if (lane == 0) {
    DLf[s_abs] += wf * (dotf + dl);
    const float cn = wn * donon - wn * (dotn + dl);
    corrn[s_abs] = cn;
    if (corrn_dense) corrn_dense[wid] = cn;
    lsen[s_abs] = lse_n[wid];
  }
}

// End of a cell's backward.  do_c / dlse_c: gradient of the committed-prefix partial summed over the
// cell's sweeps (dense [B, R, H, DH] / [B, R, H]); o_c / lse_c: the partial itself; dK0 / dV0: gradient
// of the rows sweep 0 read (the raw rows).  Writes, at the cell's rows of the per-layer arrays indexed by
// absolute position (batch strides bs_vec / bs_sca): doc = d o_c (compute dtype), corr = d o_c . o_c -
// d lse_c (also as a dense [B, R, H] copy for the query-side kernel), lsec = lse_c; and adds dK0 / dV0
// into the raw-row gradients dks / dv.
template <int DH, typename TD>
__global__ void __launch_bounds__(256) cell_finish_kernel(
    const float* __restrict__ do_c, const float* __restrict__ dlse_c, const float* __restrict__ o_c,
    const float* __restrict__ lse_c, const float* __restrict__ dK0, const float* __restrict__ dV0,
    TD* __restrict__ doc, float* __restrict__ corr, float* __restrict__ corr_dense, float* __restrict__ lsec,
    float* __restrict__ dks, float* __restrict__ dv, long long bs_vec, long long bs_sca, int B, int R, int H) {
  const long long wid = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (wid >= (long long)B * R * H) return;
  const int h = (int)(wid % H);
  const long long br = wid / H;
  const int r = (int)(br % R), b = (int)(br / R);
  const long long s_abs = (long long)b * bs_sca + (long long)r * H + h;
  const long long v_abs = (long long)b * bs_vec + ((long long)r * H + h) * DH;
  constexpr int PER = DH / 32;
  float dot = 0.f, g[PER], oc[PER], k0[PER], v0[PER], ak[PER], av_[PER];
  ldf<PER>(do_c + wid * DH + lane * PER, g);
  ldf<PER>(o_c + wid * DH + lane * PER, oc);
  ldf<PER>(dK0 + wid * DH + lane * PER, k0);
  ldf<PER>(dV0 + wid * DH + lane * PER, v0);
  ldf<PER>(dks + v_abs + lane * PER, ak);
  ldf<PER>(dv + v_abs + lane * PER, av_);
#pragma unroll
  for (int e = 0; e < PER; ++e) {
    dot += g[e] * oc[e];
    ak[e] += k0[e];
    av_[e] += v0[e];
  }
  stv<PER>(doc + v_abs + lane * PER, g);
  stf<PER>(dks + v_abs + lane * PER, ak);
  stf<PER>(dv + v_abs + lane * PER, av_);
  dot = warp_sum(dot);
  if (lane == 0) {
    const float cv = dot - dlse_c[wid];
    corr[s_abs] = cv;
    corr_dense[wid] = cv;
    lsec[s_abs] = lse_c[wid];
  }
}

// End of a cell's backward when the sweeps deferred their row-scalar x row products (tail backward in DEFER
// mode).  sp.dO[k]: the gradient of sweep k's read, dense [B, R, H, DH] fp32; scal: [K][3][B*R*H] = (p_self, p_c,
// delta) of every sweep.  q, ks, vr: the cell's rotated query, raw rotated key and raw value rows (bf16 views with
// their own batch / row strides).  Forms, per (row, head):
//   d v_raw  += sum_k p_self,k dO_k + dV0          d o_c = sum_k p_c,k dO_k   (-> doc in the compute dtype)
//   dss       = sum_k p_self,k (dO_k . v_raw - delta_k) scale
//   d k_self += dss q + dK0                        d q  += dss k_self
//   d lse_c   = sum_k p_c,k (dO_k . o_c - delta_k)   corr = d o_c . o_c - d lse_c,   lsec = lse_c
// Sweeps are summed in the order the reverse pass met them (k = K-1 first).
struct SweepPtrs {
  const float* dO[64];
};

// KT > 0: the sweep count as a compile-time constant (the loop unrolls and every sweep's loads are issued up front)
template <int DH, typename TD, int KT>
__global__ void __launch_bounds__(256) cell_finish_sweeps_kernel(
    SweepPtrs sp, int K, const float* __restrict__ scal, const bf16* __restrict__ q, TView vq,
    const bf16* __restrict__ ks, TView vks, const bf16* __restrict__ vr, TView vvr, const float* __restrict__ o_c, const float* __restrict__ lse_c,
    const float* __restrict__ dK0, const float* __restrict__ dV0, TD* __restrict__ doc, float* __restrict__ corr,
    float* __restrict__ corr_dense, float* __restrict__ lsec, float* __restrict__ dks, float* __restrict__ dv,
    float* __restrict__ dq, float scale, long long bs_vec, long long bs_sca, int B, int R, int H) {
  // DH = 64: half a warp per (batch, row, head), 16 bytes per lane; DH = 128: a warp, 16 bytes per lane.  Lanes past
  // the end stay in the shuffles (clamped to the last unit) and store nothing.
  constexpr int LPH = DH == 64 ? 16 : 32, PER = DH / LPH;
  const long long n = (long long)B * R * H;
  const long long unit = ((long long)blockIdx.x * blockDim.x + threadIdx.x) / LPH;
  const bool live = unit < n;
  const long long wid = live ? unit : n - 1;
  const int lane = threadIdx.x & (LPH - 1);
  const int h = (int)(wid % H);
  const long long br = wid / H;
  const int r = (int)(br % R), b = (int)(br / R);
  const long long s_abs = (long long)b * bs_sca + (long long)r * H + h;
  const long long v_abs = (long long)b * bs_vec + ((long long)r * H + h) * DH;
  const bf16* q_row = q + b * vq.bs + r * vq.rs + (long long)h * DH;
  const bf16* ks_row = ks + b * vks.bs + r * vks.rs + (long long)h * DH;
  const bf16* vr_row = vr + b * vvr.bs + r * vvr.rs + (long long)h * DH;
  float vv[PER], oc[PER], av[PER], ac[PER];
  ldb<PER>(vr_row + lane * PER, vv);
  ldf<PER>(o_c + wid * DH + lane * PER, oc);
#pragma unroll
  for (int e = 0; e < PER; ++e) av[e] = ac[e] = 0.f;
  float dss = 0.f, dl = 0.f;
  const int Kn = KT > 0 ? KT : K;
#pragma unroll
  for (int kk = 0; kk < Kn; ++kk) {
    const int k = Kn - 1 - kk;
    const float* sc = scal + (long long)k * 3 * n + wid;
    const float ps = sc[0], pc = sc[n], delta = sc[2 * n];
    float g[PER], dsv = 0.f, dc = 0.f;
    ldf<PER>(sp.dO[k] + wid * DH + lane * PER, g);
#pragma unroll
    for (int e = 0; e < PER; ++e) {
      dsv += g[e] * vv[e];
      dc += g[e] * oc[e];
      av[e] += ps * g[e];
      ac[e] += pc * g[e];
    }
#pragma unroll
    for (int o = LPH / 2; o > 0; o >>= 1) {
      dsv += __shfl_xor_sync(0xffffffffu, dsv, o);
      dc += __shfl_xor_sync(0xffffffffu, dc, o);
    }
    dss += ps * (dsv - delta) * scale;
    dl += pc * (dc - delta);
  }
  float dot = 0.f, qv[PER], kv[PER], k0[PER], v0[PER], a_k[PER], a_v[PER], a_q[PER];
  ldb<PER>(q_row + lane * PER, qv);
  ldb<PER>(ks_row + lane * PER, kv);
  ldf<PER>(dK0 + wid * DH + lane * PER, k0);
  ldf<PER>(dV0 + wid * DH + lane * PER, v0);
  ldf<PER>(dks + v_abs + lane * PER, a_k);
  ldf<PER>(dv + v_abs + lane * PER, a_v);
  ldf<PER>(dq + v_abs + lane * PER, a_q);
#pragma unroll
  for (int e = 0; e < PER; ++e) {
    dot += ac[e] * oc[e];
    a_k[e] += k0[e] + dss * qv[e];
    a_v[e] += v0[e] + av[e];
    a_q[e] += dss * kv[e];
  }
#pragma unroll
  for (int o = LPH / 2; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
  if (!live) return;
  stv<PER>(doc + v_abs + lane * PER, ac);
  stf<PER>(dks + v_abs + lane * PER, a_k);
  stf<PER>(dv + v_abs + lane * PER, a_v);
  stf<PER>(dq + v_abs + lane * PER, a_q);
  if (lane == 0) {
    const float cv = dot - dl;
    corr[s_abs] = cv;
    corr_dense[wid] = cv;
    lsec[s_abs] = lse_c[wid];
  }
}

// End of a wavefront chunk's backward (every sweep of the chunk has been processed).  The arrays are indexed by
// absolute position and start at the chunk's first row (batch strides bs_vec / bs_sca).  The far read's
// accumulated gradient (DOf, DLf) becomes what the prefix backward kernels consume: doc = DOf (compute dtype),
// corr = DOf . o_f - DLf (also dense [B, R, H]), lsec = lse_f (also dense); the pending gradient of the rows the
// chunk's first sweep read (its raw rows) moves into the raw-row gradients: dks += dKp, dv += dVp, dKp = dVp = 0.
// With K > 0 the raw-row gradients of the chunk's K sweeps were deferred (tail backward, mode 2): sweep k left its
// d o rows (sw.dO[k], batch stride sw.bs_vec[k]) and per-(row, head) scalars p_self (sw.ps[k]) and dss (sw.dss[k],
// batch stride sw.bs_sca[k]); here dv += sum_k p_self,k dO_k and dks += (sum_k dss_k) q (q: the chunk's rotated
// query rows, bf16 view).  With `dglx` the gates' x-logit gradient of the chunk's rows is formed here as well: it
// equals, sweep by sweep, the gate columns [2d, 4d) of the stashed d(ctx / gate logits) (sw.dcg[k]), so it is
// summed over the K sweeps once and written (fp32 [B, R, 2d] view, batch stride bs_dglx) instead of being
// read-modify-written by every step's refine backward.
struct ChunkSweeps {
  const float* dO[64];
  const float* ps[64];
  const float* dss[64];
  const bf16* dcg[64];      // optional: the sweep's stashed d(ctx / gate logits) rows [B, R, 4d] (batch stride 4 bs_vec)
  long long bs_vec[64];
  long long bs_sca[64];
};

// KT > 0: the sweep count as a compile-time constant (the loop unrolls and every sweep's loads are issued up front)
template <int DH, typename TD, int KT>
__global__ void __launch_bounds__(256) chunk_finish_kernel(
    const float* __restrict__ DOf, const float* __restrict__ DLf, const float* __restrict__ o_f,
    const float* __restrict__ lse_f, float* __restrict__ dKp, float* __restrict__ dVp, float* __restrict__ dks,
    float* __restrict__ dv, TD* __restrict__ doc, float* __restrict__ corr, float* __restrict__ lsec,
    float* __restrict__ corr_dense, float* __restrict__ lse_dense, long long bs_vec, long long bs_sca, int B, int R,
    int H, const __grid_constant__ ChunkSweeps sw, int K, const bf16* __restrict__ q, TView vq,
    float* __restrict__ dglx, long long bs_dglx) {
  const long long wid = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (wid >= (long long)B * R * H) return;
  const int h = (int)(wid % H);
  const long long br = wid / H;
  const int r = (int)(br % R), b = (int)(br / R);
  const long long s_abs = (long long)b * bs_sca + (long long)r * H + h;
  const long long v_abs = (long long)b * bs_vec + ((long long)r * H + h) * DH;
  constexpr int PER = DH / 32;
  float av[PER], agk[PER], agv[PER], dss = 0.f;
#pragma unroll
  for (int e = 0; e < PER; ++e) av[e] = agk[e] = agv[e] = 0.f;
  const long long d = (long long)H * DH;
  const int Kn = KT > 0 ? KT : K;
#pragma unroll
  for (int kk = 0; kk < Kn; ++kk) {
    const int k = Kn - 1 - kk;
    const long long so = (long long)b * sw.bs_sca[k] + (long long)r * H + h;
    const float ps = sw.ps[k][so];
    dss += sw.dss[k][so];
    float g[PER];
    ldf<PER>(sw.dO[k] + (long long)b * sw.bs_vec[k] + ((long long)r * H + h) * DH + lane * PER, g);
#pragma unroll
    for (int e = 0; e < PER; ++e) av[e] += ps * g[e];
    if (dglx) {
      const bf16* c_ = sw.dcg[k] + (long long)b * 4 * sw.bs_vec[k] + (long long)r * 4 * d + 2 * d + (long long)h * DH;
      float gk[PER], gv[PER];
      ldb<PER>(c_ + lane * PER, gk);
      ldb<PER>(c_ + d + lane * PER, gv);
#pragma unroll
      for (int e = 0; e < PER; ++e) {
        agk[e] += gk[e];
        agv[e] += gv[e];
      }
    }
  }
  if (dglx) {
    float* o_ = dglx + (long long)b * bs_dglx + (long long)r * 2 * d + (long long)h * DH;
    stf<PER>(o_ + lane * PER, agk);
    stf<PER>(o_ + d + lane * PER, agv);
  }
  float dot = 0.f, g[PER], of[PER], kp[PER], vp[PER], a_k[PER], a_v[PER], qv[PER], zero[PER];
#pragma unroll
  for (int e = 0; e < PER; ++e) qv[e] = zero[e] = 0.f;
  if (K > 0) ldb<PER>(q + b * vq.bs + r * vq.rs + (long long)h * DH + lane * PER, qv);
  ldf<PER>(DOf + v_abs + lane * PER, g);
  ldf<PER>(o_f + v_abs + lane * PER, of);
  ldf<PER>(dKp + v_abs + lane * PER, kp);
  ldf<PER>(dVp + v_abs + lane * PER, vp);
  ldf<PER>(dks + v_abs + lane * PER, a_k);
  ldf<PER>(dv + v_abs + lane * PER, a_v);
#pragma unroll
  for (int e = 0; e < PER; ++e) {
    dot += g[e] * of[e];
    a_k[e] += kp[e] + dss * qv[e];
    a_v[e] += vp[e] + av[e];
  }
  stv<PER>(doc + v_abs + lane * PER, g);
  stf<PER>(dks + v_abs + lane * PER, a_k);
  stf<PER>(dv + v_abs + lane * PER, a_v);
  stf<PER>(dKp + v_abs + lane * PER, zero);
  stf<PER>(dVp + v_abs + lane * PER, zero);
  dot = warp_sum(dot);
  if (lane == 0) {
    const float cv = dot - DLf[s_abs], l = lse_f[s_abs];
    corr[s_abs] = cv;
    corr_dense[wid] = cv;
    lsec[s_abs] = l;
    lse_dense[wid] = l;
  }
}

// Two block copies of the same geometry in one launch: [B, n16] 16-byte words each, per-tensor batch strides.
__global__ void __launch_bounds__(256) copy_pair_kernel(const uint4* __restrict__ s0, uint4* __restrict__ d0,
                                                        const uint4* __restrict__ s1, uint4* __restrict__ d1,
                                                        long long sbs, long long dbs, long long n16) {
  const uint4* s = (blockIdx.z ? s1 : s0) + (long long)blockIdx.y * sbs;
  uint4* d = (blockIdx.z ? d1 : d0) + (long long)blockIdx.y * dbs;
  const long long step = (long long)gridDim.x * blockDim.x;
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  for (; i + 3 * step < n16; i += 4 * step) {
    const uint4 a = s[i], b = s[i + step], c = s[i + 2 * step], e = s[i + 3 * step];
    d[i] = a;
    d[i + step] = b;
    d[i + 2 * step] = c;
    d[i + 3 * step] = e;
  }
  for (; i < n16; i += step) d[i] = s[i];
}

}  // namespace

extern "C" {

int dmb_cell_finish(const float* do_c, const float* dlse_c, const float* o_c, const float* lse_c, const float* dK0,
                    const float* dV0, void* doc, int doc_bf16, float* corr, float* corr_dense, float* lsec, float* dks,
                    float* dv,
                    long long bs_vec, long long bs_sca, int B, int R, int H, int DH, cudaStream_t st) {
  const long long warps = (long long)B * R * H;
  const unsigned blocks = (unsigned)((warps * 32 + 255) / 256);
#define GO(D, T)                                                                                            \
  cell_finish_kernel<D, T><<<blocks, 256, 0, st>>>(do_c, dlse_c, o_c, lse_c, dK0, dV0, (T*)doc, corr,       \
                                                   corr_dense, lsec, dks, dv, bs_vec, bs_sca, B, R, H)
  if (DH == 64) {
    if (doc_bf16) GO(64, bf16); else GO(64, float);
  } else if (DH == 128) {
    if (doc_bf16) GO(128, bf16); else GO(128, float);
  } else {
    return -1;
  }
#undef GO
  DMB_CHECK_LAUNCH();
  return 0;
}

int dmb_wave_merge_fwd(const float* o_f, const float* lse_f, long long bs_vec, long long bs_sca, const float* o_n,
                       const float* lse_n, float* o_c, float* lse_c, float* w_f, float* w_n, int B, int R, int H,
                       int DH, cudaStream_t st) {
  const long long warps = (long long)B * R * H;
  const unsigned blocks = (unsigned)((warps * 32 + 255) / 256);
  if (DH == 64)
    merge_fwd_kernel<64><<<blocks, 256, 0, st>>>(o_f, lse_f, bs_vec, bs_sca, o_n, lse_n, o_c, lse_c, w_f, w_n, B, R, H);
  else if (DH == 128)
    merge_fwd_kernel<128><<<blocks, 256, 0, st>>>(o_f, lse_f, bs_vec, bs_sca, o_n, lse_n, o_c, lse_c, w_f, w_n, B, R, H);
  else
    return -1;
  DMB_CHECK_LAUNCH();
  return 0;
}

// docn_bf16: 1 = the near d o buffer is bf16, 0 = fp32
int dmb_wave_split_bwd(const float* do_c, const float* dlse_c, const float* o_c, const float* o_n, const float* lse_n,
                       const float* w_f, const float* w_n, const float* o_f, float* DOf, float* DLf, void* docn,
                       int docn_bf16, float* corrn, float* corrn_dense, float* lsen, long long bs_vec, long long bs_sca,
                       int B, int R, int H, int DH, cudaStream_t st) {
  const long long warps = (long long)B * R * H;
  const unsigned blocks = (unsigned)((warps * 32 + 255) / 256);
#define GO(D, T)                                                                                              \
  split_bwd_kernel<D, T><<<blocks, 256, 0, st>>>(do_c, dlse_c, o_c, o_n, lse_n, w_f, w_n, o_f, DOf, DLf,      \
                                                 (T*)docn, corrn, corrn_dense, lsen, bs_vec, bs_sca, B, R, H)
  if (DH == 64) {
    if (docn_bf16) GO(64, bf16); else GO(64, float);
  } else if (DH == 128) {
    if (docn_bf16) GO(128, bf16); else GO(128, float);
  } else {
    return -1;
  }
#undef GO
  DMB_CHECK_LAUNCH();
  return 0;
}

// dO_ptrs: K host-side pointers (K <= 64) to the sweeps' dense fp32 gradients
int dmb_cell_finish_sweeps(const float* const* dO_ptrs, int K, const float* scal, const void* q, TView vq,
                           const void* ks, TView vks, const void* vr, TView vvr, const float* o_c, const float* lse_c, const float* dK0, const float* dV0,
                           void* doc, int doc_bf16, float* corr, float* corr_dense, float* lsec, float* dks, float* dv,
                           float* dq, float scale, long long bs_vec, long long bs_sca, int B, int R, int H, int DH,
                           cudaStream_t st) {
  if (K < 1 || K > 64) return -1;
  SweepPtrs sp;
  for (int k = 0; k < 64; ++k) sp.dO[k] = dO_ptrs[k < K ? k : K - 1];
  const long long lanes = (long long)B * R * H * (DH == 64 ? 16 : 32);
  const unsigned blocks = (unsigned)((lanes + 255) / 256);
#define GO(D, T)                                                                                                    \
  do {                                                                                                              \
    if (K == 4)                                                                                                     \
      cell_finish_sweeps_kernel<D, T, 4><<<blocks, 256, 0, st>>>(sp, K, scal, (const bf16*)q, vq, (const bf16*)ks, vks, \
          (const bf16*)vr, vvr, o_c, lse_c, dK0, dV0, (T*)doc, corr, corr_dense, lsec, dks, dv, dq, scale, bs_vec,   \
          bs_sca, B, R, H);                                                                                         \
    else                                                                                                            \
      cell_finish_sweeps_kernel<D, T, 0><<<blocks, 256, 0, st>>>(sp, K, scal, (const bf16*)q, vq, (const bf16*)ks, vks, \
          (const bf16*)vr, vvr, o_c, lse_c, dK0, dV0, (T*)doc, corr, corr_dense, lsec, dks, dv, dq, scale, bs_vec,   \
          bs_sca, B, R, H);                                                                                         \
  } while (0)
  if (DH == 64) {
    if (doc_bf16) GO(64, bf16); else GO(64, float);
  } else if (DH == 128) {
    if (doc_bf16) GO(128, bf16); else GO(128, float);
  } else {
    return -1;
  }
#undef GO
  DMB_CHECK_LAUNCH();
  return 0;
}

// sweeps: K (0..64) deferred sweeps; dO_ptrs / ps_ptrs / dss_ptrs (/ dcg_ptrs when dglx is given) and the two stride
// arrays have K entries (host)
int dmb_wave_chunk_finish(const float* DOf, const float* DLf, const float* o_f, const float* lse_f, float* dKp,
                          float* dVp, float* dks, float* dv, void* doc, int doc_bf16, float* corr, float* lsec,
                          float* corr_dense, float* lse_dense, long long bs_vec, long long bs_sca, int B, int R, int H,
                          int DH, int K, const float* const* dO_ptrs, const float* const* ps_ptrs,
                          const float* const* dss_ptrs, const long long* sw_bs_vec, const long long* sw_bs_sca,
                          const void* q, TView vq, const void* const* dcg_ptrs, float* dglx, long long bs_dglx,
                          cudaStream_t st) {
  if (K < 0 || K > 64) return -1;
  ChunkSweeps sw = {};
  for (int k = 0; k < K; ++k) {
    sw.dO[k] = dO_ptrs[k];
    sw.ps[k] = ps_ptrs[k];
    sw.dss[k] = dss_ptrs[k];
    sw.dcg[k] = dglx ? (const bf16*)dcg_ptrs[k] : nullptr;
    sw.bs_vec[k] = sw_bs_vec[k];
    sw.bs_sca[k] = sw_bs_sca[k];
  }
  const long long warps = (long long)B * R * H;
  const unsigned blocks = (unsigned)((warps * 32 + 255) / 256);
#define GO(D, T)                                                                                                 \
  do {                                                                                                           \
    if (K == 8)                                                                                                  \
      chunk_finish_kernel<D, T, 8><<<blocks, 256, 0, st>>>(DOf, DLf, o_f, lse_f, dKp, dVp, dks, dv, (T*)doc, corr, \
          lsec, corr_dense, lse_dense, bs_vec, bs_sca, B, R, H, sw, K, (const bf16*)q, vq, dglx, bs_dglx);       \
    else                                                                                                         \
      chunk_finish_kernel<D, T, 0><<<blocks, 256, 0, st>>>(DOf, DLf, o_f, lse_f, dKp, dVp, dks, dv, (T*)doc, corr, \
          lsec, corr_dense, lse_dense, bs_vec, bs_sca, B, R, H, sw, K, (const bf16*)q, vq, dglx, bs_dglx);       \
  } while (0)
  if (DH == 64) {
    if (doc_bf16) GO(64, bf16); else GO(64, float);
  } else if (DH == 128) {
    if (doc_bf16) GO(128, bf16); else GO(128, float);
  } else {
    return -1;
  }
#undef GO
  DMB_CHECK_LAUNCH();
  return 0;
}

// src / dst: 16-byte aligned, row_bytes a multiple of 16; strides in bytes (multiples of 16).
int dmb_copy_pair(const void* s0, void* d0, const void* s1, void* d1, long long src_bs, long long dst_bs,
                  long long row_bytes, int B, cudaStream_t st) {
  if ((row_bytes | src_bs | dst_bs) & 15) return -1;
  const long long n16 = row_bytes >> 4;
  long long bx = (n16 + 256 * 4 - 1) / (256 * 4);
  if (bx < 1) bx = 1;
  if (bx > 1024) bx = 1024;
  dim3 grid((unsigned)bx, (unsigned)B, 2);
  copy_pair_kernel<<<grid, 256, 0, st>>>((const uint4*)s0, (uint4*)d0, (const uint4*)s1, (uint4*)d1, src_bs >> 4,
                                         dst_bs >> 4, n16);
  DMB_CHECK_LAUNCH();
  return 0;
}

}  // extern "C"
