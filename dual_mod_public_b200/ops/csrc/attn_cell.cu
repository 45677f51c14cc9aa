// Chunk-cell attention kernels: committed-prefix pass and per-sweep tail read, forward and
// backward.  One CTA per (batch, head); C/16 warps, each owning 16 query rows.  Tiles live in
// padded shared memory and go through warp-level bf16 tensor-core MMAs with fp32 softmax.
//
// Read algebra (per chunk row i, all in fp32):
//   lse = log( exp(lse_c) + sum_{j<i} exp(s_ij) + exp(s_self) ),  o = P_c o_c + sum_j P_j v_j + P_self v_raw
// and its hand-derived backward; see engines/fused_math.py for the plain-torch statement.
#include "attn_tiles.cuh"

using namespace attn;

namespace {

// =============================================================================================
// tail forward
// =============================================================================================
// Groups (gridDim.z > 1): one launch covers G consecutive chunks of the same sequences.  Strided tensors
// (slices of [B, T, ...] buffers) advance `grow` rows per group; dense tensors are [B, G, C, ...]
// (equivalently [B, G*C, ...]), indexed with bd = b * G + group.
template <int DH, int C>
__global__ void __launch_bounds__(C * 2) tail_fwd_kernel(
    const bf16* __restrict__ q, TView vq, const bf16* __restrict__ ks, TView vks,
    const bf16* __restrict__ vr, TView vvr, const bf16* __restrict__ Kin, TView vKin,
    const bf16* __restrict__ Vin, TView vVin, const float* __restrict__ o_c,
    const float* __restrict__ lse_c, bf16* __restrict__ o, float* __restrict__ lse,
    float* __restrict__ ssq, int H, float scale, int window, int grow) {
  constexpr int P = Tile<DH>::PITCH, NT = C * 2, NB = C / 8;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* sQ = reinterpret_cast<bf16*>(smem_raw);
  bf16* sK = sQ + C * P;
  bf16* sV = sK + C * P;
  const int h = blockIdx.x, b = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int bd = b * gridDim.z + blockIdx.z;
  {
    const long long go = (long long)blockIdx.z * grow;
    q += go * vq.rs; ks += go * vks.rs; vr += go * vvr.rs; Kin += go * vKin.rs; Vin += go * vVin.rs;
  }
  const int g = lane >> 2, t = lane & 3;
  const long long hoff = (long long)h * DH;
  load_tile_bf16<DH, NT>(sQ, q + b * vq.bs + hoff, vq.rs, C, tid);
  load_tile_bf16<DH, NT>(sK, Kin + b * vKin.bs + hoff, vKin.rs, C, tid);
  load_tile_bf16<DH, NT>(sV, Vin + b * vVin.bs + hoff, vVin.rs, C, tid);
  __syncthreads();

  const int row0 = warp * 16;
  const int nb_lim = 2 * (warp + 1);  // key blocks that can hold j < i for this warp's rows
  float S[NB][4];
#pragma unroll
  for (int n = 0; n < NB; ++n) S[n][0] = S[n][1] = S[n][2] = S[n][3] = 0.f;
#pragma unroll
  for (int k0 = 0; k0 < DH; k0 += 16) {
    uint32_t a[4];
    load_a<P>(a, sQ, row0, k0, lane);
#pragma unroll
    for (int n = 0; n < NB; n += 2) {
      if (n < nb_lim) {
        uint32_t bb[4];
        load_b_nk<P>(bb, sK, n * 8, k0, lane);
        mma16816(S[n], a, bb[0], bb[1]);
        mma16816(S[n + 1], a, bb[2], bb[3]);
      }
    }
  }
  // rows owned by this thread: i0 = row0 + g, i1 = i0 + 8
  const int i0 = row0 + g, i1 = i0 + 8;
  const long long orow0 = ((long long)(bd * C + i0) * H + h), orow1 = ((long long)(bd * C + i1) * H + h);
  float ss0 = quad_dot_bf16<DH>(sQ + i0 * P, ks + b * vks.bs + i0 * vks.rs + hoff, t) * scale;
  float ss1 = quad_dot_bf16<DH>(sQ + i1 * P, ks + b * vks.bs + i1 * vks.rs + hoff, t) * scale;
  const float lc0 = lse_c[orow0], lc1 = lse_c[orow1];
  float m0 = fmaxf(ss0, lc0), m1 = fmaxf(ss1, lc1);
#pragma unroll
  for (int n = 0; n < NB; ++n) {
    int j = n * 8 + 2 * t;
    S[n][0] = intra_ok(i0, j, window) ? S[n][0] * scale : -INFINITY;
    S[n][1] = intra_ok(i0, j + 1, window) ? S[n][1] * scale : -INFINITY;
    S[n][2] = intra_ok(i1, j, window) ? S[n][2] * scale : -INFINITY;
    S[n][3] = intra_ok(i1, j + 1, window) ? S[n][3] * scale : -INFINITY;
    m0 = fmaxf(m0, fmaxf(S[n][0], S[n][1]));
    m1 = fmaxf(m1, fmaxf(S[n][2], S[n][3]));
  }
  m0 = quad_max(m0);
  m1 = quad_max(m1);
  float z0 = 0.f, z1 = 0.f;
#pragma unroll
  for (int n = 0; n < NB; ++n) {
    S[n][0] = __expf(S[n][0] - m0);
    S[n][1] = __expf(S[n][1] - m0);
    S[n][2] = __expf(S[n][2] - m1);
    S[n][3] = __expf(S[n][3] - m1);
    z0 += S[n][0] + S[n][1];
    z1 += S[n][2] + S[n][3];
  }
  z0 = quad_sum(z0);
  z1 = quad_sum(z1);
  const float es0 = __expf(ss0 - m0), es1 = __expf(ss1 - m1);
  const float ec0 = __expf(lc0 - m0), ec1 = __expf(lc1 - m1);
  z0 += es0 + ec0;
  z1 += es1 + ec1;
  // O = P V
  float O[DH / 8][4];
#pragma unroll
  for (int n = 0; n < DH / 8; ++n) O[n][0] = O[n][1] = O[n][2] = O[n][3] = 0.f;
#pragma unroll
  for (int kk = 0; kk < C / 16; ++kk) {
    if (2 * kk < nb_lim) {
      uint32_t a[4] = {pack_bf16(S[2 * kk][0], S[2 * kk][1]), pack_bf16(S[2 * kk][2], S[2 * kk][3]),
                       pack_bf16(S[2 * kk + 1][0], S[2 * kk + 1][1]),
                       pack_bf16(S[2 * kk + 1][2], S[2 * kk + 1][3])};
#pragma unroll
      for (int n = 0; n < DH / 8; n += 2) {
        uint32_t bb[4];
        load_b_kn<P>(bb, sV, kk * 16, n * 8, lane);
        mma16816(O[n], a, bb[0], bb[1]);
        mma16816(O[n + 1], a, bb[2], bb[3]);
      }
    }
  }
  const float r0 = 1.f / z0, r1 = 1.f / z1;
  const bf16* vr0 = vr + b * vvr.bs + i0 * vvr.rs + hoff;
  const bf16* vr1 = vr + b * vvr.bs + i1 * vvr.rs + hoff;
  const float* oc0 = o_c + orow0 * DH;
  const float* oc1 = o_c + orow1 * DH;
  bf16* out0 = o + orow0 * DH;
  bf16* out1 = o + orow1 * DH;
  float sq0 = 0.f, sq1 = 0.f;
#pragma unroll
  for (int n = 0; n < DH / 8; ++n) {
    int d = n * 8 + 2 * t;
    float2 v0 = __bfloat1622float2(*reinterpret_cast<const bf162*>(vr0 + d));
    float2 v1 = __bfloat1622float2(*reinterpret_cast<const bf162*>(vr1 + d));
    float2 c0 = *reinterpret_cast<const float2*>(oc0 + d);
    float2 c1 = *reinterpret_cast<const float2*>(oc1 + d);
    const float a0 = (O[n][0] + es0 * v0.x + ec0 * c0.x) * r0, a1 = (O[n][1] + es0 * v0.y + ec0 * c0.y) * r0;
    const float b0 = (O[n][2] + es1 * v1.x + ec1 * c1.x) * r1, b1 = (O[n][3] + es1 * v1.y + ec1 * c1.y) * r1;
    sq0 += a0 * a0 + a1 * a1;
    sq1 += b0 * b0 + b1 * b1;
    *reinterpret_cast<bf162*>(out0 + d) = __floats2bfloat162_rn(a0, a1);
    *reinterpret_cast<bf162*>(out1 + d) = __floats2bfloat162_rn(b0, b1);
  }
  sq0 = quad_sum(sq0);
  sq1 = quad_sum(sq1);
  if (t == 0) {
    lse[orow0] = m0 + __logf(z0);
    lse[orow1] = m1 + __logf(z1);
    ssq[orow0] = sq0;      // per-head sum of squares of the read: the row norm needs no pass over o
    ssq[orow1] = sq1;
  }
}

// =============================================================================================
// tail backward
// =============================================================================================
// DEFER = 1: the sweep's row-scalar x row products (d v_raw = p_self dO, d o_c = p_c dO, the self-column terms and
// d lse_c) are left to the cell-end kernel, which forms them for all sweeps of the cell at once from the kept dO
// rows; this kernel then only stashes (p_self, p_c, delta) per (row, head) in `dlsec_acc` = [3][rows] and touches
// neither dks_acc, dv_acc, doc_acc nor v_raw / o_c.
// DEFER = 2: only the raw-row gradients are left to the chunk-end kernel (d v_raw = sum p_self dO, d k_self = (sum dss) q):
// dv_acc is not touched and `dks_acc` receives the stash [2][rows] = (p_self, dss); d q, d o_c, d lse_c as in mode 0.
template <int DH, int C, int DEFER>
__global__ void __launch_bounds__(C * 2, DH <= 64 ? 4 : 2) tail_bwd_kernel(
    const float* __restrict__ dO, const bf16* __restrict__ q, TView vq, const bf16* __restrict__ ks,
    TView vks, const bf16* __restrict__ vr, TView vvr, const bf16* __restrict__ Kin, TView vKin,
    const bf16* __restrict__ Vin, TView vVin, const float* __restrict__ o_c,
    const float* __restrict__ lse_c, const bf16* __restrict__ o, const float* __restrict__ lse,
    float* __restrict__ dq_acc, TView vdq, float* __restrict__ dks_acc, TView vdks, float* __restrict__ dv_acc,
    TView vdv, float* __restrict__ doc_acc, float* __restrict__ dlsec_acc, float* __restrict__ dKin,
    float* __restrict__ dVin, TView vdkin, int H, float scale, int window, int grow, int flags) {
  // flags: bit 0 = dq_acc is written instead of added to; bit 1 = the same for doc_acc / dlsec_acc (the
  // first sweep processed of a cell initialises its accumulators, so nobody has to zero them).  dq_acc and
  // dKin / dVin are (batch stride, row stride) views: they may be windows of [B, T, h, dh] arrays.
  const bool init_dq = flags & 1, init_doc = flags & 2;
  constexpr int P = Tile<DH>::PITCH, NT = C * 2, NB = C / 8, PC = C + 8;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* sQ = reinterpret_cast<bf16*>(smem_raw);
  bf16* sK = sQ + C * P;
  bf16* sV = sK + C * P;
  bf16* sdO = sV + C * P;
  bf16* sP = sdO + C * P;
  bf16* sdS = sP + C * PC;
  const int h = blockIdx.x, b = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const long long hoff = (long long)h * DH;
  const int bd = b * gridDim.z + blockIdx.z;
  {
    const long long go = (long long)blockIdx.z * grow;
    q += go * vq.rs; ks += go * vks.rs; vr += go * vvr.rs; Kin += go * vKin.rs; Vin += go * vVin.rs;
    dks_acc += go * vdks.rs; dv_acc += go * vdv.rs; dq_acc += go * vdq.rs; dKin += go * vdkin.rs; dVin += go * vdkin.rs;
  }
  const long long dense_rs = (long long)H * DH;  // contiguous [B,C,H,DH] tensors
  const long long dense_b = (long long)bd * C * dense_rs + hoff;
  const int row0 = warp * 16, nb_lim = 2 * (warp + 1);
  const int i0 = row0 + g, i1 = i0 + 8;
  // per-row scalars first (self score, delta = dO.o, dO.v_raw, dO.o_c): their global loads are in flight
  // together with the tile loads below instead of sitting between the two MMA phases
  const long long orow0 = ((long long)(bd * C + i0) * H + h), orow1 = ((long long)(bd * C + i1) * H + h);
  const float* dO0 = dO + orow0 * DH;
  const float* dO1 = dO + orow1 * DH;
  const bf16* ks0 = ks + b * vks.bs + i0 * vks.rs + hoff;
  const bf16* ks1 = ks + b * vks.bs + i1 * vks.rs + hoff;
  const bf16* vr0 = vr + b * vvr.bs + i0 * vvr.rs + hoff;
  const bf16* vr1 = vr + b * vvr.bs + i1 * vvr.rs + hoff;
  const float L0 = lse[orow0], L1 = lse[orow1];
  const float ss0 = quad_dot_bf16<DH>(q + b * vq.bs + i0 * vq.rs + hoff, ks0, t) * scale;
  const float ss1 = quad_dot_bf16<DH>(q + b * vq.bs + i1 * vq.rs + hoff, ks1, t) * scale;
  const float ps0 = __expf(ss0 - L0), ps1 = __expf(ss1 - L1);
  const float pc0 = __expf(lse_c[orow0] - L0), pc1 = __expf(lse_c[orow1] - L1);
  const float delta0 = quad_dot_f32_bf16<DH>(dO0, o + orow0 * DH, t);
  const float delta1 = quad_dot_f32_bf16<DH>(dO1, o + orow1 * DH, t);
  float dss0 = 0.f, dss1 = 0.f;
  if constexpr (DEFER == 1) {
    if (t == 0) {
      const long long n_rows = (long long)gridDim.y * gridDim.z * C * H;
      dlsec_acc[orow0] = ps0; dlsec_acc[n_rows + orow0] = pc0; dlsec_acc[2 * n_rows + orow0] = delta0;
      dlsec_acc[orow1] = ps1; dlsec_acc[n_rows + orow1] = pc1; dlsec_acc[2 * n_rows + orow1] = delta1;
    }
  } else {
    const float dsv0 = quad_dot_f32_bf16<DH>(dO0, vr0, t), dsv1 = quad_dot_f32_bf16<DH>(dO1, vr1, t);
    const float doc0 = quad_dot_f32<DH>(dO0, o_c + orow0 * DH, t);
    const float doc1 = quad_dot_f32<DH>(dO1, o_c + orow1 * DH, t);
    dss0 = ps0 * (dsv0 - delta0) * scale;
    dss1 = ps1 * (dsv1 - delta1) * scale;
    if (t == 0) {
      dlsec_acc[orow0] = (init_doc ? 0.f : dlsec_acc[orow0]) + pc0 * (doc0 - delta0);
      dlsec_acc[orow1] = (init_doc ? 0.f : dlsec_acc[orow1]) + pc1 * (doc1 - delta1);
      if constexpr (DEFER == 2) {
        const long long n_rows = (long long)gridDim.y * gridDim.z * C * H;
        dks_acc[orow0] = ps0; dks_acc[n_rows + orow0] = dss0;
        dks_acc[orow1] = ps1; dks_acc[n_rows + orow1] = dss1;
      }
    }
  }
  load_tile_bf16<DH, NT>(sQ, q + b * vq.bs + hoff, vq.rs, C, tid);
  load_tile_bf16<DH, NT>(sK, Kin + b * vKin.bs + hoff, vKin.rs, C, tid);
  load_tile_bf16<DH, NT>(sV, Vin + b * vVin.bs + hoff, vVin.rs, C, tid);
  load_tile_f32<DH, NT>(sdO, dO + dense_b, dense_rs, C, tid);
  __syncthreads();

  float S[NB][4], dP[NB][4];
#pragma unroll
  for (int n = 0; n < NB; ++n) {
    S[n][0] = S[n][1] = S[n][2] = S[n][3] = 0.f;
    dP[n][0] = dP[n][1] = dP[n][2] = dP[n][3] = 0.f;
  }
#pragma unroll
  for (int k0 = 0; k0 < DH; k0 += 16) {
    uint32_t a[4], ad[4];
    load_a<P>(a, sQ, row0, k0, lane);
    load_a<P>(ad, sdO, row0, k0, lane);
#pragma unroll
    for (int n = 0; n < NB; n += 2) {
      if (n < nb_lim) {
        uint32_t bb[4];
        load_b_nk<P>(bb, sK, n * 8, k0, lane);
        mma16816(S[n], a, bb[0], bb[1]);
        mma16816(S[n + 1], a, bb[2], bb[3]);
        load_b_nk<P>(bb, sV, n * 8, k0, lane);
        mma16816(dP[n], ad, bb[0], bb[1]);
        mma16816(dP[n + 1], ad, bb[2], bb[3]);
      }
    }
  }
  // P and dS for the intra block (zero where masked or skipped), kept as bf16 A-fragments and in smem
#pragma unroll
  for (int n = 0; n < NB; ++n) {
    int j = n * 8 + 2 * t;
    float p0 = intra_ok(i0, j, window) ? __expf(S[n][0] * scale - L0) : 0.f;
    float p1 = intra_ok(i0, j + 1, window) ? __expf(S[n][1] * scale - L0) : 0.f;
    float p2 = intra_ok(i1, j, window) ? __expf(S[n][2] * scale - L1) : 0.f;
    float p3 = intra_ok(i1, j + 1, window) ? __expf(S[n][3] * scale - L1) : 0.f;
    S[n][0] = p0; S[n][1] = p1; S[n][2] = p2; S[n][3] = p3;
    dP[n][0] = p0 * (dP[n][0] - delta0) * scale;
    dP[n][1] = p1 * (dP[n][1] - delta0) * scale;
    dP[n][2] = p2 * (dP[n][2] - delta1) * scale;
    dP[n][3] = p3 * (dP[n][3] - delta1) * scale;
    *reinterpret_cast<uint32_t*>(sP + i0 * PC + j) = pack_bf16(p0, p1);
    *reinterpret_cast<uint32_t*>(sP + i1 * PC + j) = pack_bf16(p2, p3);
    *reinterpret_cast<uint32_t*>(sdS + i0 * PC + j) = pack_bf16(dP[n][0], dP[n][1]);
    *reinterpret_cast<uint32_t*>(sdS + i1 * PC + j) = pack_bf16(dP[n][2], dP[n][3]);
  }
  // dQ = dS K_in  (+ self column)
  float A[DH / 8][4];
#pragma unroll
  for (int n = 0; n < DH / 8; ++n) A[n][0] = A[n][1] = A[n][2] = A[n][3] = 0.f;
#pragma unroll
  for (int kk = 0; kk < C / 16; ++kk) {
    if (2 * kk < nb_lim) {
      uint32_t a[4] = {pack_bf16(dP[2 * kk][0], dP[2 * kk][1]), pack_bf16(dP[2 * kk][2], dP[2 * kk][3]),
                       pack_bf16(dP[2 * kk + 1][0], dP[2 * kk + 1][1]),
                       pack_bf16(dP[2 * kk + 1][2], dP[2 * kk + 1][3])};
#pragma unroll
      for (int n = 0; n < DH / 8; n += 2) {
        uint32_t bb[4];
        load_b_kn<P>(bb, sK, kk * 16, n * 8, lane);
        mma16816(A[n], a, bb[0], bb[1]);
        mma16816(A[n + 1], a, bb[2], bb[3]);
      }
    }
  }
  if constexpr (DEFER == 1) {
    float* dq0 = dq_acc + b * vdq.bs + i0 * vdq.rs + hoff;
    float* dq1 = dq_acc + b * vdq.bs + i1 * vdq.rs + hoff;
#pragma unroll
    for (int n = 0; n < DH / 8; ++n) {
      const int d = n * 8 + 2 * t;
      float2 x = init_dq ? make_float2(0.f, 0.f) : *reinterpret_cast<float2*>(dq0 + d);
      x.x += A[n][0]; x.y += A[n][1];
      *reinterpret_cast<float2*>(dq0 + d) = x;
      x = init_dq ? make_float2(0.f, 0.f) : *reinterpret_cast<float2*>(dq1 + d);
      x.x += A[n][2]; x.y += A[n][3];
      *reinterpret_cast<float2*>(dq1 + d) = x;
    }
  } else {
    float* dq0 = dq_acc + b * vdq.bs + i0 * vdq.rs + hoff;
    float* dq1 = dq_acc + b * vdq.bs + i1 * vdq.rs + hoff;
    float* dk0 = dks_acc + b * vdks.bs + i0 * vdks.rs + hoff;
    float* dk1 = dks_acc + b * vdks.bs + i1 * vdks.rs + hoff;
    float* dv0 = dv_acc + b * vdv.bs + i0 * vdv.rs + hoff;
    float* dv1 = dv_acc + b * vdv.bs + i1 * vdv.rs + hoff;
    float* dc0 = doc_acc + orow0 * DH;
    float* dc1 = doc_acc + orow1 * DH;
#pragma unroll
    for (int n = 0; n < DH / 8; ++n) {
      int d = n * 8 + 2 * t;
      float2 k0v = __bfloat1622float2(*reinterpret_cast<const bf162*>(ks0 + d));
      float2 k1v = __bfloat1622float2(*reinterpret_cast<const bf162*>(ks1 + d));
      float2 q0v = __bfloat1622float2(*reinterpret_cast<const bf162*>(sQ + i0 * P + d));
      float2 q1v = __bfloat1622float2(*reinterpret_cast<const bf162*>(sQ + i1 * P + d));
      float2 g0 = *reinterpret_cast<const float2*>(dO0 + d);
      float2 g1 = *reinterpret_cast<const float2*>(dO1 + d);
      float2 x;
      x = init_dq ? make_float2(0.f, 0.f) : *reinterpret_cast<float2*>(dq0 + d);
      x.x += A[n][0] + dss0 * k0v.x; x.y += A[n][1] + dss0 * k0v.y;
      *reinterpret_cast<float2*>(dq0 + d) = x;
      x = init_dq ? make_float2(0.f, 0.f) : *reinterpret_cast<float2*>(dq1 + d);
      x.x += A[n][2] + dss1 * k1v.x; x.y += A[n][3] + dss1 * k1v.y;
      *reinterpret_cast<float2*>(dq1 + d) = x;
      if constexpr (DEFER == 0) {
        x = *reinterpret_cast<float2*>(dk0 + d);
        x.x += dss0 * q0v.x; x.y += dss0 * q0v.y;
        *reinterpret_cast<float2*>(dk0 + d) = x;
        x = *reinterpret_cast<float2*>(dk1 + d);
        x.x += dss1 * q1v.x; x.y += dss1 * q1v.y;
        *reinterpret_cast<float2*>(dk1 + d) = x;
        x = *reinterpret_cast<float2*>(dv0 + d);
        x.x += ps0 * g0.x; x.y += ps0 * g0.y;
        *reinterpret_cast<float2*>(dv0 + d) = x;
        x = *reinterpret_cast<float2*>(dv1 + d);
        x.x += ps1 * g1.x; x.y += ps1 * g1.y;
        *reinterpret_cast<float2*>(dv1 + d) = x;
      }
      x = init_doc ? make_float2(0.f, 0.f) : *reinterpret_cast<float2*>(dc0 + d);
      x.x += pc0 * g0.x; x.y += pc0 * g0.y;
      *reinterpret_cast<float2*>(dc0 + d) = x;
      x = init_doc ? make_float2(0.f, 0.f) : *reinterpret_cast<float2*>(dc1 + d);
      x.x += pc1 * g1.x; x.y += pc1 * g1.y;
      *reinterpret_cast<float2*>(dc1 + d) = x;
    }
  }
  __syncthreads();
  // dK_in = dS^T Q, dV_in = P^T dO : this warp owns keys [row0, row0+16); queries > key only
  float GK[DH / 8][4], GV[DH / 8][4];
#pragma unroll
  for (int n = 0; n < DH / 8; ++n) {
    GK[n][0] = GK[n][1] = GK[n][2] = GK[n][3] = 0.f;
    GV[n][0] = GV[n][1] = GV[n][2] = GV[n][3] = 0.f;
  }
#pragma unroll
  for (int kk = 0; kk < C / 16; ++kk) {
    if (kk >= warp) {
      uint32_t as[4], ap[4];
      load_a_t<PC>(as, sdS, row0, kk * 16, lane);
      load_a_t<PC>(ap, sP, row0, kk * 16, lane);
#pragma unroll
      for (int n = 0; n < DH / 8; n += 2) {
        uint32_t bb[4];
        load_b_kn<P>(bb, sQ, kk * 16, n * 8, lane);
        mma16816(GK[n], as, bb[0], bb[1]);
        mma16816(GK[n + 1], as, bb[2], bb[3]);
        load_b_kn<P>(bb, sdO, kk * 16, n * 8, lane);
        mma16816(GV[n], ap, bb[0], bb[1]);
        mma16816(GV[n + 1], ap, bb[2], bb[3]);
      }
    }
  }
  float* gk0 = dKin + b * vdkin.bs + i0 * vdkin.rs + hoff;
  float* gk1 = dKin + b * vdkin.bs + i1 * vdkin.rs + hoff;
  float* gv0 = dVin + b * vdkin.bs + i0 * vdkin.rs + hoff;
  float* gv1 = dVin + b * vdkin.bs + i1 * vdkin.rs + hoff;
#pragma unroll
  for (int n = 0; n < DH / 8; ++n) {
    int d = n * 8 + 2 * t;
    *reinterpret_cast<float2*>(gk0 + d) = make_float2(GK[n][0], GK[n][1]);
    *reinterpret_cast<float2*>(gk1 + d) = make_float2(GK[n][2], GK[n][3]);
    *reinterpret_cast<float2*>(gv0 + d) = make_float2(GV[n][0], GV[n][1]);
    *reinterpret_cast<float2*>(gv1 + d) = make_float2(GV[n][2], GV[n][3]);
  }
}

// =============================================================================================
// committed-prefix forward: chunk queries against tape rows [lo, pos0)
// =============================================================================================

template <int DH, int C>
__global__ void __launch_bounds__(C * 2, DH <= 64 ? 4 : 2) prefix_fwd_kernel(
    const bf16* __restrict__ q, TView vq, const bf16* __restrict__ Kc, const bf16* __restrict__ Vc,
    TView vc, float* __restrict__ o_c, float* __restrict__ lse_c, int H, int lo, int pos0,
    float scale, int window, int grow, int qoff) {
  constexpr int P = Tile<DH>::PITCH, NT = C * 2, NB = KT / 8;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* sQ = reinterpret_cast<bf16*>(smem_raw);
  bf16* sK = sQ + C * P;        // 2 stages
  bf16* sV = sK + 2 * KT * P;   // 2 stages
  const int h = blockIdx.x, b = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int bd = b * gridDim.z + blockIdx.z;
  // group z reads the tape rows [max(0, lo + z * grow), pos0 + z * grow) for the queries of chunk z
  q += (long long)blockIdx.z * grow * vq.rs;
  pos0 += blockIdx.z * grow;
  lo = max(0, lo + (int)blockIdx.z * grow);
  // query row t sits at absolute position pos0 + qoff + t (qoff > 0: the key range ends before the chunk);
  // with a sliding window no row can see a key before qpos - window + 1
  const int qpos = pos0 + qoff;
  if (window) lo = min(pos0, max(lo, qpos - window + 1));
  const int g = lane >> 2, t = lane & 3;
  const long long hoff = (long long)h * DH;
  const bf16* Kb = Kc + b * vc.bs + hoff;
  const bf16* Vb = Vc + b * vc.bs + hoff;
  const int n_keys = pos0 - lo, n_tiles = (n_keys + KT - 1) / KT;
  load_tile_bf16<DH, NT>(sQ, q + b * vq.bs + hoff, vq.rs, C, tid);
  auto issue = [&](int tile, int stage) {
    int k0 = lo + tile * KT, rows = min(KT, pos0 - k0);
    load_tile_async<DH, NT>(sK + stage * KT * P, Kb + (long long)k0 * vc.rs, vc.rs, rows, tid);
    load_tile_async<DH, NT>(sV + stage * KT * P, Vb + (long long)k0 * vc.rs, vc.rs, rows, tid);
    cp_async_commit();
    if (rows < KT) {  // rows past the prefix get probability 0; keep their V finite
      constexpr int CH = DH / 8;
      for (int i = tid; i < (KT - rows) * CH; i += NT) {
        int r = rows + i / CH, c = (i % CH) * 8;
        *reinterpret_cast<uint4*>(sK + (stage * KT + r) * P + c) = make_uint4(0, 0, 0, 0);
        *reinterpret_cast<uint4*>(sV + (stage * KT + r) * P + c) = make_uint4(0, 0, 0, 0);
      }
    }
  };
  if (n_tiles > 0) issue(0, 0);
  const int row0 = warp * 16, i0 = row0 + g, i1 = i0 + 8;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  float O[DH / 8][4];
#pragma unroll
  for (int n = 0; n < DH / 8; ++n) O[n][0] = O[n][1] = O[n][2] = O[n][3] = 0.f;
  for (int tile = 0; tile < n_tiles; ++tile) {
    const int stage = tile & 1;
    if (tile + 1 < n_tiles) {
      issue(tile + 1, stage ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const bf16* tK = sK + stage * KT * P;
    const bf16* tV = sV + stage * KT * P;
    const int kbase = lo + tile * KT, rows = min(KT, pos0 - kbase);
    float S[NB][4];
#pragma unroll
    for (int n = 0; n < NB; ++n) S[n][0] = S[n][1] = S[n][2] = S[n][3] = 0.f;
#pragma unroll
    for (int k0 = 0; k0 < DH; k0 += 16) {
      uint32_t a[4];
      load_a<P>(a, sQ, row0, k0, lane);
#pragma unroll
      for (int n = 0; n < NB; n += 2) {
        uint32_t bb[4];
        load_b_nk<P>(bb, tK, n * 8, k0, lane);
        mma16816(S[n], a, bb[0], bb[1]);
        mma16816(S[n + 1], a, bb[2], bb[3]);
      }
    }
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int n = 0; n < NB; ++n) {
      int jl = n * 8 + 2 * t, j = kbase + jl;
      bool in0 = jl < rows, in1 = jl + 1 < rows;
      bool a0 = in0 && (window == 0 || j > qpos + i0 - window);
      bool a1 = in1 && (window == 0 || j + 1 > qpos + i0 - window);
      bool a2 = in0 && (window == 0 || j > qpos + i1 - window);
      bool a3 = in1 && (window == 0 || j + 1 > qpos + i1 - window);
      S[n][0] = a0 ? S[n][0] * scale : -INFINITY;
      S[n][1] = a1 ? S[n][1] * scale : -INFINITY;
      S[n][2] = a2 ? S[n][2] * scale : -INFINITY;
      S[n][3] = a3 ? S[n][3] * scale : -INFINITY;
      mx0 = fmaxf(mx0, fmaxf(S[n][0], S[n][1]));
      mx1 = fmaxf(mx1, fmaxf(S[n][2], S[n][3]));
    }
    mx0 = quad_max(mx0);
    mx1 = quad_max(mx1);
    const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
    const float sub0 = (mn0 == -INFINITY) ? 0.f : mn0, sub1 = (mn1 == -INFINITY) ? 0.f : mn1;
    const float c0 = __expf(m0 - sub0), c1 = __expf(m1 - sub1);  // exp(-inf)=0 on the first tile
    m0 = mn0;
    m1 = mn1;
    float z0 = 0.f, z1 = 0.f;
#pragma unroll
    for (int n = 0; n < NB; ++n) {
      S[n][0] = __expf(S[n][0] - sub0);
      S[n][1] = __expf(S[n][1] - sub0);
      S[n][2] = __expf(S[n][2] - sub1);
      S[n][3] = __expf(S[n][3] - sub1);
      z0 += S[n][0] + S[n][1];
      z1 += S[n][2] + S[n][3];
    }
    l0 = l0 * c0 + quad_sum(z0);
    l1 = l1 * c1 + quad_sum(z1);
#pragma unroll
    for (int n = 0; n < DH / 8; ++n) {
      O[n][0] *= c0; O[n][1] *= c0; O[n][2] *= c1; O[n][3] *= c1;
    }
#pragma unroll
    for (int kk = 0; kk < KT / 16; ++kk) {
      uint32_t a[4] = {pack_bf16(S[2 * kk][0], S[2 * kk][1]), pack_bf16(S[2 * kk][2], S[2 * kk][3]),
                       pack_bf16(S[2 * kk + 1][0], S[2 * kk + 1][1]),
                       pack_bf16(S[2 * kk + 1][2], S[2 * kk + 1][3])};
      if (kk * 16 < rows) {
#pragma unroll
        for (int n = 0; n < DH / 8; n += 2) {
          uint32_t bb[4];
          load_b_kn<P>(bb, tV, kk * 16, n * 8, lane);
          mma16816(O[n], a, bb[0], bb[1]);
          mma16816(O[n + 1], a, bb[2], bb[3]);
        }
      }
    }
    __syncthreads();
  }
  const long long orow0 = ((long long)(bd * C + i0) * H + h), orow1 = ((long long)(bd * C + i1) * H + h);
  const float r0 = l0 > 0.f ? 1.f / l0 : 0.f, r1 = l1 > 0.f ? 1.f / l1 : 0.f;
  float* out0 = o_c + orow0 * DH;
  float* out1 = o_c + orow1 * DH;
#pragma unroll
  for (int n = 0; n < DH / 8; ++n) {
    int d = n * 8 + 2 * t;
    *reinterpret_cast<float2*>(out0 + d) = make_float2(O[n][0] * r0, O[n][1] * r0);
    *reinterpret_cast<float2*>(out1 + d) = make_float2(O[n][2] * r1, O[n][3] * r1);
  }
  if (t == 0) {
    lse_c[orow0] = l0 > 0.f ? m0 + __logf(l0) : DMB_NEG;
    lse_c[orow1] = l1 > 0.f ? m1 + __logf(l1) : DMB_NEG;
  }
}

}  // namespace

extern "C" {

int dmb_tail_fwd(const void* q, TView vq, const void* ks, TView vks, const void* vr, TView vvr,
                 const void* Kin, TView vKin, const void* Vin, TView vVin, const float* o_c,
                 const float* lse_c, void* o, float* lse, float* ssq, int B, int c, int H, int dh,
                 float scale, int window, int G, int grow, cudaStream_t st) {
  DISPATCH_DH_C(dh, c, {
    size_t smem = (size_t)3 * C * Tile<DH>::PITCH * sizeof(bf16);
    auto kern = tail_fwd_kernel<DH, C>;
    if (set_smem(kern, smem)) return -2;
    kern<<<dim3(H, B, G), C * 2, smem, st>>>((const bf16*)q, vq, (const bf16*)ks, vks, (const bf16*)vr, vvr,
                                            (const bf16*)Kin, vKin, (const bf16*)Vin, vVin, o_c, lse_c,
                                            (bf16*)o, lse, ssq, H, scale, window, grow);
  })
  DMB_CHECK_LAUNCH();
  return 0;
}

int dmb_tail_bwd(const float* dO, const void* q, TView vq, const void* ks, TView vks, const void* vr,
                 TView vvr, const void* Kin, TView vKin, const void* Vin, TView vVin,
                 const float* o_c, const float* lse_c, const void* o, const float* lse, float* dq_acc,
                 TView vdq, float* dks_acc, TView vdks, float* dv_acc, TView vdv, float* doc_acc,
                 float* dlsec_acc, float* dKin, float* dVin, TView vdkin, int B, int c, int H, int dh, float scale,
                 int window, int G, int grow, int flags, cudaStream_t st) {
  DISPATCH_DH_C(dh, c, {
    size_t smem = ((size_t)4 * C * Tile<DH>::PITCH + (size_t)2 * C * (C + 8)) * sizeof(bf16);
    if (flags & 8) {
      auto kern = tail_bwd_kernel<DH, C, 2>;
      if (set_smem(kern, smem)) return -2;
      kern<<<dim3(H, B, G), C * 2, smem, st>>>(dO, (const bf16*)q, vq, (const bf16*)ks, vks, (const bf16*)vr,
                                              vvr, (const bf16*)Kin, vKin, (const bf16*)Vin, vVin, o_c,
                                              lse_c, (const bf16*)o, lse, dq_acc, vdq, dks_acc, vdks, dv_acc, vdv,
                                              doc_acc, dlsec_acc, dKin, dVin, vdkin, H, scale, window, grow, flags);
    } else if (flags & 4) {
      auto kern = tail_bwd_kernel<DH, C, 1>;
      if (set_smem(kern, smem)) return -2;
      kern<<<dim3(H, B, G), C * 2, smem, st>>>(dO, (const bf16*)q, vq, (const bf16*)ks, vks, (const bf16*)vr,
                                              vvr, (const bf16*)Kin, vKin, (const bf16*)Vin, vVin, o_c,
                                              lse_c, (const bf16*)o, lse, dq_acc, vdq, dks_acc, vdks, dv_acc, vdv,
                                              doc_acc, dlsec_acc, dKin, dVin, vdkin, H, scale, window, grow, flags);
    } else {
      auto kern = tail_bwd_kernel<DH, C, 0>;
      if (set_smem(kern, smem)) return -2;
      kern<<<dim3(H, B, G), C * 2, smem, st>>>(dO, (const bf16*)q, vq, (const bf16*)ks, vks, (const bf16*)vr,
                                              vvr, (const bf16*)Kin, vKin, (const bf16*)Vin, vVin, o_c,
                                              lse_c, (const bf16*)o, lse, dq_acc, vdq, dks_acc, vdks, dv_acc, vdv,
                                              doc_acc, dlsec_acc, dKin, dVin, vdkin, H, scale, window, grow, flags);
    }
  })
  DMB_CHECK_LAUNCH();
  return 0;
}

int dmb_prefix_fwd(const void* q, TView vq, const void* Kc, const void* Vc, TView vc, float* o_c,
                   float* lse_c, int B, int c, int H, int dh, int lo, int pos0, float scale,
                   int window, int G, int grow, int qoff, cudaStream_t st) {
  DISPATCH_DH_C(dh, c, {
    size_t smem = ((size_t)C + 4 * KT) * Tile<DH>::PITCH * sizeof(bf16);
    auto kern = prefix_fwd_kernel<DH, C>;
    if (set_smem(kern, smem)) return -2;
    kern<<<dim3(H, B, G), C * 2, smem, st>>>((const bf16*)q, vq, (const bf16*)Kc, (const bf16*)Vc, vc, o_c,
                                         lse_c, H, lo, pos0, scale, window, grow, qoff);
  })
  DMB_CHECK_LAUNCH();
  return 0;
}

}  // extern "C"
