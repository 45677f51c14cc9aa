// Backward of the committed-prefix read, owner-computes on both sides: no gradient is ever
// accumulated in global memory across launches.
//
//   prefix_dkv : one CTA owns the C tape rows of a chunk for one (batch, head) and walks over every
//                LATER query row of the sequence (all of them read this chunk through their prefix
//                pass), accumulating dK / dV of its rows in registers; written once.
//   prefix_dq  : one CTA owns the C query rows of a cell and walks over its committed prefix,
//                accumulating dq in registers.
//
// Both recompute P = exp(s - lse_c) from the saved per-row log-sum-exp and use
//   dS = P * (d o_c . v - corr) * scale,   corr = d o_c . o_c - d lse_c   (per query row),
// where d o_c (bf16) and corr (fp32) of every row are laid out by absolute position.
#include "attn_tiles.cuh"

using namespace attn;

namespace {

// ---------------------------------------------------------------------------------------------
// key side.  q_all / doc_all: [B, T, H, DH] bf16 (dense);  corr_all / lsec_all: [B, T, H] fp32.
// Tape rows [pos0, pos0 + C) of Kc / Vc;  queries t in [q_start, T).
template <int DH, int C>
__global__ void __launch_bounds__(C * 2, DH <= 64 ? 4 : 2) prefix_dkv_kernel(
    const bf16* __restrict__ q_all, const bf16* __restrict__ doc_all, const float* __restrict__ corr_all,
    const float* __restrict__ lsec_all, const bf16* __restrict__ Kc, const bf16* __restrict__ Vc, TView vc,
    float* __restrict__ dK, float* __restrict__ dV, TView vdkv, int accumulate, int T, int H, int pos0, int q_start,
    int q_end, float scale, int window, int grow, int span) {
  constexpr int P = Tile<DH>::PITCH, NT = C * 2, NB = C / 8, PC = C + 8, QT = C;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* sK = reinterpret_cast<bf16*>(smem_raw);
  bf16* sV = sK + C * P;
  // ST stages of query / d o_c tiles: one at head dim 64, so that four CTAs fit an SM (the other CTAs
  // cover the load latency), two at head dim 128 where registers allow two CTAs anyway
  constexpr int ST = DH <= 64 ? 1 : 2;
  bf16* sQ = sV + C * P;            // ST stages of [QT][P]
  bf16* sdO = sQ + ST * QT * P;     // ST stages
  bf16* sP = sdO + ST * QT * P;     // [QT][PC]
  bf16* sdS = sP + QT * PC;
  const int h = blockIdx.x, b = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t4 = lane & 3;
  // groups (gridDim.z > 1): key chunk z of a run of consecutive chunks; its readers are the query rows
  // [max(q_start, chunk end), min(q_end, chunk start + span)); outputs are dense [B, G, C, H, DH]
  pos0 += blockIdx.z * grow;
  q_start = max(q_start, pos0 + C);
  q_end = min(q_end, pos0 + span);
  const long long hoff = (long long)h * DH, rs = (long long)H * DH;
  const bf16* Qb = q_all + (long long)b * T * rs + hoff;
  const bf16* Ob = doc_all + (long long)b * T * rs + hoff;
  const float* Lb = lsec_all + (long long)b * T * H + h;
  const float* Cb = corr_all + (long long)b * T * H + h;
  load_tile_bf16<DH, NT>(sK, Kc + b * vc.bs + (long long)pos0 * vc.rs + hoff, vc.rs, C, tid);
  load_tile_bf16<DH, NT>(sV, Vc + b * vc.bs + (long long)pos0 * vc.rs + hoff, vc.rs, C, tid);
  const int n_rows = q_end - q_start, n_tiles = (n_rows + QT - 1) / QT;
  auto issue = [&](int tile, int stage) {
    const int t0 = q_start + tile * QT, rows = min(QT, q_end - t0);
    load_tile_async<DH, NT>(sQ + stage * QT * P, Qb + (long long)t0 * rs, rs, rows, tid);
    load_tile_async<DH, NT>(sdO + stage * QT * P, Ob + (long long)t0 * rs, rs, rows, tid);
    cp_async_commit();
    if (rows < QT) {  // rows past the sequence end get probability 0; keep their operands finite
      constexpr int CH = DH / 8;
      for (int i = tid; i < (QT - rows) * CH; i += NT) {
        int r = rows + i / CH, c = (i % CH) * 8;
        *reinterpret_cast<uint4*>(sQ + (stage * QT + r) * P + c) = make_uint4(0, 0, 0, 0);
        *reinterpret_cast<uint4*>(sdO + (stage * QT + r) * P + c) = make_uint4(0, 0, 0, 0);
      }
    }
  };
  if (n_tiles > 0) issue(0, 0);
  const int row0 = warp * 16;
  float GK[DH / 8][4], GV[DH / 8][4];
#pragma unroll
  for (int n = 0; n < DH / 8; ++n) {
    GK[n][0] = GK[n][1] = GK[n][2] = GK[n][3] = 0.f;
    GV[n][0] = GV[n][1] = GV[n][2] = GV[n][3] = 0.f;
  }
  for (int tile = 0; tile < n_tiles; ++tile) {
    const int stage = ST == 2 ? (tile & 1) : 0;
    if (ST == 2 && tile + 1 < n_tiles) {
      issue(tile + 1, stage ^ 1);
      cp_async_wait<1>();
    } else {
      if (ST == 1 && tile > 0) issue(tile, 0);       // the single buffer was released by the sync below
      cp_async_wait<0>();
    }
    __syncthreads();
    const bf16* tQ = sQ + stage * QT * P;
    const bf16* tO = sdO + stage * QT * P;
    const int t0 = q_start + tile * QT;
    // ---- phase 1: this warp's 16 query rows against the C keys
    float S[NB][4], dP[NB][4];
#pragma unroll
    for (int n = 0; n < NB; ++n) {
      S[n][0] = S[n][1] = S[n][2] = S[n][3] = 0.f;
      dP[n][0] = dP[n][1] = dP[n][2] = dP[n][3] = 0.f;
    }
#pragma unroll
    for (int k0 = 0; k0 < DH; k0 += 16) {
      uint32_t a[4], ad[4];
      load_a<P>(a, tQ, row0, k0, lane);
      load_a<P>(ad, tO, row0, k0, lane);
#pragma unroll
      for (int n = 0; n < NB; n += 2) {
        uint32_t bb[4];
        load_b_nk<P>(bb, sK, n * 8, k0, lane);
        mma16816(S[n], a, bb[0], bb[1]);
        mma16816(S[n + 1], a, bb[2], bb[3]);
        load_b_nk<P>(bb, sV, n * 8, k0, lane);
        mma16816(dP[n], ad, bb[0], bb[1]);
        mma16816(dP[n + 1], ad, bb[2], bb[3]);
      }
    }
    const int i0 = row0 + g, i1 = i0 + 8;             // rows inside the tile
    const int ta = t0 + i0, tb = t0 + i1;             // absolute query positions
    const bool va = ta < q_end, vb = tb < q_end;
    const float L0 = va ? Lb[(long long)ta * H] : 0.f, L1 = vb ? Lb[(long long)tb * H] : 0.f;
    const float c0 = va ? Cb[(long long)ta * H] : 0.f, c1 = vb ? Cb[(long long)tb * H] : 0.f;
#pragma unroll
    for (int n = 0; n < NB; ++n) {
      const int jl = n * 8 + 2 * t4, j = pos0 + jl;
      const bool a0 = va && (window == 0 || j > ta - window), a1 = va && (window == 0 || j + 1 > ta - window);
      const bool a2 = vb && (window == 0 || j > tb - window), a3 = vb && (window == 0 || j + 1 > tb - window);
      const float p0 = a0 ? __expf(S[n][0] * scale - L0) : 0.f, p1 = a1 ? __expf(S[n][1] * scale - L0) : 0.f;
      const float p2 = a2 ? __expf(S[n][2] * scale - L1) : 0.f, p3 = a3 ? __expf(S[n][3] * scale - L1) : 0.f;
      *reinterpret_cast<uint32_t*>(sP + i0 * PC + jl) = pack_bf16(p0, p1);
      *reinterpret_cast<uint32_t*>(sP + i1 * PC + jl) = pack_bf16(p2, p3);
      *reinterpret_cast<uint32_t*>(sdS + i0 * PC + jl) =
          pack_bf16(p0 * (dP[n][0] - c0) * scale, p1 * (dP[n][1] - c0) * scale);
      *reinterpret_cast<uint32_t*>(sdS + i1 * PC + jl) =
          pack_bf16(p2 * (dP[n][2] - c1) * scale, p3 * (dP[n][3] - c1) * scale);
    }
    __syncthreads();
    // ---- phase 2: this warp's 16 keys gather from all QT query rows
#pragma unroll
    for (int kk = 0; kk < QT / 16; ++kk) {
      uint32_t as[4], ap[4];
      load_a_t<PC>(as, sdS, row0, kk * 16, lane);
      load_a_t<PC>(ap, sP, row0, kk * 16, lane);
#pragma unroll
      for (int n = 0; n < DH / 8; n += 2) {
        uint32_t bb[4];
        load_b_kn<P>(bb, tQ, kk * 16, n * 8, lane);
        mma16816(GK[n], as, bb[0], bb[1]);
        mma16816(GK[n + 1], as, bb[2], bb[3]);
        load_b_kn<P>(bb, tO, kk * 16, n * 8, lane);
        mma16816(GV[n], ap, bb[0], bb[1]);
        mma16816(GV[n + 1], ap, bb[2], bb[3]);
      }
    }
    __syncthreads();   // sP / sdS and this stage's tiles are free again
  }
  // outputs: (batch stride, row stride) views, group z at rows [z * grow, z * grow + C); added to when
  // `accumulate` (the rows may be a window of a pending-gradient array)
  const int ka = row0 + g, kb = ka + 8;
  const long long ob = b * vdkv.bs + (long long)blockIdx.z * grow * vdkv.rs + hoff;
  float* outs[4] = {dK + ob + ka * vdkv.rs, dK + ob + kb * vdkv.rs, dV + ob + ka * vdkv.rs, dV + ob + kb * vdkv.rs};
#pragma unroll
  for (int n = 0; n < DH / 8; ++n) {
    const int d = n * 8 + 2 * t4;
    float2 vals[4] = {make_float2(GK[n][0], GK[n][1]), make_float2(GK[n][2], GK[n][3]),
                      make_float2(GV[n][0], GV[n][1]), make_float2(GV[n][2], GV[n][3])};
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      if (accumulate) {
        const float2 o = *reinterpret_cast<const float2*>(outs[u] + d);
        vals[u].x += o.x; vals[u].y += o.y;
      }
      *reinterpret_cast<float2*>(outs[u] + d) = vals[u];
    }
  }
}

// ---------------------------------------------------------------------------------------------
// query side for one cell.  q: [B, C, H, DH] view; do_c: bf16 view with the same strides class;
// lse_c / corr: dense [B, C, H] fp32; dq_acc: dense [B, C, H, DH] fp32, accumulated into.
template <int DH, int C>
__global__ void __launch_bounds__(C * 2, DH <= 64 ? 4 : 2) prefix_dq_kernel(
    const bf16* __restrict__ q, TView vq, const bf16* __restrict__ do_c, TView vdo,
    const bf16* __restrict__ Kc, const bf16* __restrict__ Vc, TView vc, const float* __restrict__ lse_c,
    const float* __restrict__ corr, float* __restrict__ dq_acc, TView vdq, int H, int lo, int pos0, float scale,
    int window, int grow, int qoff) {
  constexpr int P = Tile<DH>::PITCH, NT = C * 2, NB = KT / 8;
  constexpr int ST = 2;            // key / value tiles are double-buffered
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* sQ = reinterpret_cast<bf16*>(smem_raw);
  bf16* sdO = sQ + C * P;
  bf16* sK = sdO + C * P;        // 2 stages
  bf16* sV = sK + 2 * KT * P;    // 2 stages
  const int h = blockIdx.x, b = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t4 = lane & 3;
  // groups (gridDim.z > 1): chunk z of the same sequences; strided tensors advance `grow` rows per group,
  // dense ones are [B, G, C, ...]; the key range is [max(0, lo + z * grow), pos0 + z * grow)
  const int bd = b * gridDim.z + blockIdx.z;
  q += (long long)blockIdx.z * grow * vq.rs;
  do_c += (long long)blockIdx.z * grow * vdo.rs;
  pos0 += blockIdx.z * grow;
  lo = max(0, lo + (int)blockIdx.z * grow);
  const int qpos = pos0 + qoff;            // absolute position of query row 0
  if (window) lo = min(pos0, max(lo, qpos - window + 1));
  const long long hoff = (long long)h * DH;
  const bf16* Kb = Kc + b * vc.bs + hoff;
  const bf16* Vb = Vc + b * vc.bs + hoff;
  load_tile_bf16<DH, NT>(sQ, q + b * vq.bs + hoff, vq.rs, C, tid);
  load_tile_bf16<DH, NT>(sdO, do_c + b * vdo.bs + hoff, vdo.rs, C, tid);
  const int n_tiles = (pos0 - lo + KT - 1) / KT;
  auto issue = [&](int tile, int stage) {
    const int k0 = lo + tile * KT, rows = min(KT, pos0 - k0);
    load_tile_async<DH, NT>(sK + stage * KT * P, Kb + (long long)k0 * vc.rs, vc.rs, rows, tid);
    load_tile_async<DH, NT>(sV + stage * KT * P, Vb + (long long)k0 * vc.rs, vc.rs, rows, tid);
    cp_async_commit();
    if (rows < KT) {
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
  const long long orow0 = ((long long)(bd * C + i0) * H + h), orow1 = ((long long)(bd * C + i1) * H + h);
  const float L0 = lse_c[orow0], L1 = lse_c[orow1], c0 = corr[orow0], c1 = corr[orow1];
  float A[DH / 8][4];
#pragma unroll
  for (int n = 0; n < DH / 8; ++n) A[n][0] = A[n][1] = A[n][2] = A[n][3] = 0.f;
  for (int tile = 0; tile < n_tiles; ++tile) {
    const int stage = ST == 2 ? (tile & 1) : 0;
    if (ST == 2 && tile + 1 < n_tiles) {
      issue(tile + 1, stage ^ 1);
      cp_async_wait<1>();
    } else {
      if (ST == 1 && tile > 0) issue(tile, 0);       // the single buffer was released by the sync below
      cp_async_wait<0>();
    }
    __syncthreads();
    const bf16* tK = sK + stage * KT * P;
    const bf16* tV = sV + stage * KT * P;
    const int kbase = lo + tile * KT, rows = min(KT, pos0 - kbase);
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
        uint32_t bb[4];
        load_b_nk<P>(bb, tK, n * 8, k0, lane);
        mma16816(S[n], a, bb[0], bb[1]);
        mma16816(S[n + 1], a, bb[2], bb[3]);
        load_b_nk<P>(bb, tV, n * 8, k0, lane);
        mma16816(dP[n], ad, bb[0], bb[1]);
        mma16816(dP[n + 1], ad, bb[2], bb[3]);
      }
    }
#pragma unroll
    for (int n = 0; n < NB; ++n) {
      const int jl = n * 8 + 2 * t4, j = kbase + jl;
      const bool in0 = jl < rows, in1 = jl + 1 < rows;
      const bool a0 = in0 && (window == 0 || j > qpos + i0 - window);
      const bool a1 = in1 && (window == 0 || j + 1 > qpos + i0 - window);
      const bool a2 = in0 && (window == 0 || j > qpos + i1 - window);
      const bool a3 = in1 && (window == 0 || j + 1 > qpos + i1 - window);
      dP[n][0] = a0 ? __expf(S[n][0] * scale - L0) * (dP[n][0] - c0) * scale : 0.f;
      dP[n][1] = a1 ? __expf(S[n][1] * scale - L0) * (dP[n][1] - c0) * scale : 0.f;
      dP[n][2] = a2 ? __expf(S[n][2] * scale - L1) * (dP[n][2] - c1) * scale : 0.f;
      dP[n][3] = a3 ? __expf(S[n][3] * scale - L1) * (dP[n][3] - c1) * scale : 0.f;
    }
#pragma unroll
    for (int kk = 0; kk < KT / 16; ++kk) {
      if (kk * 16 < rows) {
        uint32_t a[4] = {pack_bf16(dP[2 * kk][0], dP[2 * kk][1]), pack_bf16(dP[2 * kk][2], dP[2 * kk][3]),
                         pack_bf16(dP[2 * kk + 1][0], dP[2 * kk + 1][1]),
                         pack_bf16(dP[2 * kk + 1][2], dP[2 * kk + 1][3])};
#pragma unroll
        for (int n = 0; n < DH / 8; n += 2) {
          uint32_t bb[4];
          load_b_kn<P>(bb, tK, kk * 16, n * 8, lane);
          mma16816(A[n], a, bb[0], bb[1]);
          mma16816(A[n + 1], a, bb[2], bb[3]);
        }
      }
    }
    __syncthreads();
  }
  // dq_acc: a (batch stride, row stride) view, group z at rows [z * grow, z * grow + C)
  float* dq0 = dq_acc + b * vdq.bs + ((long long)blockIdx.z * grow + i0) * vdq.rs + hoff;
  float* dq1 = dq_acc + b * vdq.bs + ((long long)blockIdx.z * grow + i1) * vdq.rs + hoff;
#pragma unroll
  for (int n = 0; n < DH / 8; ++n) {
    const int d = n * 8 + 2 * t4;
    float2 x = *reinterpret_cast<float2*>(dq0 + d);
    x.x += A[n][0]; x.y += A[n][1];
    *reinterpret_cast<float2*>(dq0 + d) = x;
    x = *reinterpret_cast<float2*>(dq1 + d);
    x.x += A[n][2]; x.y += A[n][3];
    *reinterpret_cast<float2*>(dq1 + d) = x;
  }
}

}  // namespace

extern "C" {

int dmb_prefix_dkv(const void* q_all, const void* doc_all, const float* corr_all, const float* lsec_all,
                   const void* Kc, const void* Vc, TView vc, float* dK, float* dV, TView vdkv, int accumulate, int B,
                   int T, int c, int H, int dh, int pos0, int q_start, int q_end, float scale, int window, int G,
                   int grow, int span, cudaStream_t st) {
  DISPATCH_DH_C(dh, c, {
    constexpr int ST = DH <= 64 ? 1 : 2;
    size_t smem = (((size_t)2 * C + 2 * ST * C) * Tile<DH>::PITCH + (size_t)2 * C * (C + 8)) * sizeof(bf16);
    auto kern = prefix_dkv_kernel<DH, C>;
    if (set_smem(kern, smem)) return -2;
    kern<<<dim3(H, B, G), C * 2, smem, st>>>((const bf16*)q_all, (const bf16*)doc_all, corr_all, lsec_all,
                                         (const bf16*)Kc, (const bf16*)Vc, vc, dK, dV, vdkv, accumulate, T, H, pos0,
                                         q_start, q_end < T ? q_end : T, scale, window, grow, span);
  })
  DMB_CHECK_LAUNCH();
  return 0;
}

int dmb_prefix_dq(const void* q, TView vq, const void* do_c, TView vdo, const void* Kc, const void* Vc, TView vc,
                  const float* lse_c, const float* corr, float* dq_acc, TView vdq, int B, int c, int H, int dh, int lo,
                  int pos0, float scale, int window, int G, int grow, int qoff, cudaStream_t st) {
  DISPATCH_DH_C(dh, c, {
    size_t smem = ((size_t)2 * C + 4 * KT) * Tile<DH>::PITCH * sizeof(bf16);
    auto kern = prefix_dq_kernel<DH, C>;
    if (set_smem(kern, smem)) return -2;
    kern<<<dim3(H, B, G), C * 2, smem, st>>>((const bf16*)q, vq, (const bf16*)do_c, vdo, (const bf16*)Kc,
                                         (const bf16*)Vc, vc, lse_c, corr, dq_acc, vdq, H, lo, pos0, scale, window, grow, qoff);
  })
  DMB_CHECK_LAUNCH();
  return 0;
}

}  // extern "C"
