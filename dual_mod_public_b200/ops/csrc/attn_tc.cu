// Flash-style attention forward on the 5th-generation tensor cores.
//
// One CTA per (batch, head, tile of BM query rows).  Keys and values stream from a token-major tape
// [B, T, H, DH] in tiles of 128 rows:
//
//   warp 0      TMA producer: Q once, then K / V tiles into a two-stage ring (128-byte swizzle)
//   warp 1      one thread issues  S = Q K^T  (tcgen05.mma, M = BM, N = 128, fp32 in TMEM) and
//               O_t = P V  (M = BM, N = DH) per key tile; the accumulators live in tensor memory
//   warps 2..5  softmax.  BM = 128: every thread owns one query row (its TMEM lane).  BM = 64: the
//               accumulator's 64 rows sit in lanes 0..15 of each 32-lane quarter; they are read with the
//               16-lane x 256-bit shape of tcgen05.ld, which gives every thread of the warp a warp-MMA
//               accumulator fragment (two rows, column pairs), so all 32 lanes work.  Either way the
//               threads mask, keep the running maximum and sum in the log2 domain, write
//               P = exp2(S - m) as bf16 into shared memory in the operand layout of the second
//               product (BM = 64: with stmatrix), and fold the product of the previous tile (read back
//               from TMEM, two buffers) into their fp32 output rows with the usual rescale.
//
// S of tile t+1 is issued as soon as the softmax warps have read S of tile t, so the tensor pipe works
// on the next scores and the previous P V while the exponentials run; at head dimension 64 two CTAs fit
// on an SM and fill each other's bubbles.
//
// Masking is by absolute position: query row i of group z sits at qbase + z*grow + i, key j is tape row
// j; allowed iff  lo_z <= j < hi_z,  (causal) j <= qpos - causal_excl,  (window) j > qpos - window.
// Output: o normalised (fp32 or bf16) and lse (natural log); a row without any allowed key gets o = 0
// and lse = DMB_NEG, which the merge algebra of the engines treats as an empty partial.
//
// Every mbarrier wait is bounded in time; on expiry the kernel raises a flag in global memory, stops
// waiting, lets its own copies land (bounded) and releases its tensor memory.
#include "tc05.cuh"

using namespace tc05;

namespace {

constexpr int KT = 128;                 // keys per tile
constexpr int NTHREADS = 192;

template <int DH, int BM>
struct Cfg {
  static constexpr int Q_BYTES = BM * DH * 2;
  static constexpr int KV_BYTES = KT * DH * 2;         // one K (or V) tile
  static constexpr int P_BYTES = BM * KT * 2;
  static constexpr int q_off = 0;
  static constexpr int k_off = q_off + Q_BYTES;        // 2 stages
  static constexpr int v_off = k_off + 2 * KV_BYTES;   // 2 stages
  static constexpr int p_off = v_off + 2 * KV_BYTES;
  static constexpr int bar_off = p_off + P_BYTES;
  static constexpr int total = bar_off + 256;
  static constexpr int TMEM_COLS = DH == 64 ? 256 : 512;   // S (128) + two P V buffers (2 x DH)
};

struct Geo {
  int H, Lq, lo, hi, qbase, grow, window, causal, causal_excl, tiles_q, o_bf16;
  int pshift;      // > 0 (BM = 128 only): the tile holds TWO 64-row groups; rows 64.. read keys shifted by pshift rows
  float scale_log2;
  // optional merge of this read with another partial of the same rows (o_f, lse_f: fp32, rows by absolute position
  // from the launch's first row, batch strides mf_bs_vec / mf_bs_sca): the outputs become the merged partial
  //   lse_c = log(exp(lse_f) + exp(lse_n)), o_c = w_f o_f + w_n o_n, w = exp(lse - lse_c)
  // with w_f / w_n written beside them and, when on != null, this read's own (o_n, lse_n) as well
  const float* mf_o;
  const float* mf_lse;
  long long mf_bs_vec, mf_bs_sca;
  float* m_wf;
  float* m_wn;
  float* m_on;
  float* m_lsen;
};

// one row's merge: returns lse_c and the two weights
__device__ __forceinline__ float merge_weights(float lf, float ln, float& wf, float& wn) {
  const float mm = fmaxf(lf, ln);
  const float lc = mm + __logf(__expf(lf - mm) + __expf(ln - mm));
  wf = __expf(lf - lc);
  wn = __expf(ln - lc);
  return lc;
}

template <int DH, int BM>
__global__ void __launch_bounds__(NTHREADS, (DH == 64 ? 2 : 1)) attn_fwd_tc_kernel(
    const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
    const __grid_constant__ CUtensorMap tmV, void* __restrict__ o_out, float* __restrict__ lse_out,
    const Geo g, int* __restrict__ gerr) {
  using C = Cfg<DH, BM>;
  // The swizzled tiles want a 1024-byte aligned base.  The dynamic shared window is declared with that
  // alignment instead of being padded by hand: at BM = 128, DH = 64 the padding would be what keeps a
  // second CTA off the SM.  Should a driver ever hand out a less aligned base, the kernel reports it and
  // returns before touching tensor memory or barriers.
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t base = smem_u32(smem_raw);
  if (base & 1023u) {
    if (threadIdx.x == 0) atomicExch(gerr, 2);
    return;
  }
  uint8_t* base_ptr = smem_raw;
  const uint32_t bar0 = base + C::bar_off;
  // barriers: qfull, kfull[2], vfull[2], kvempty[2], sfull, sfree, pfull, pvfull[2], pvfree[2]
  const uint32_t qfull = bar0;
  auto kfull = [&](int s) { return bar0 + 8u * (1 + s); };
  auto vfull = [&](int s) { return bar0 + 8u * (3 + s); };
  auto kvempty = [&](int s) { return bar0 + 8u * (5 + s); };
  const uint32_t sfull = bar0 + 8u * 7, sfree = bar0 + 8u * 8, pfull = bar0 + 8u * 9;
  auto pvfull = [&](int s) { return bar0 + 8u * (10 + s); };
  auto pvfree = [&](int s) { return bar0 + 8u * (12 + s); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(base_ptr + C::bar_off + 8 * 14);
  volatile int* serr = reinterpret_cast<volatile int*>(base_ptr + C::bar_off + 8 * 15);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.x, b = blockIdx.y;
  const int z = blockIdx.z / g.tiles_q, qt = blockIdx.z - z * g.tiles_q;
  // this CTA's rows and key range
  const int row0 = qt * BM, rows_here = min(BM, g.Lq - row0);
  const int lo_z = max(0, g.lo + z * g.grow), hi_z = g.hi + z * g.grow;
  const int qpos0 = g.qbase + z * g.grow + row0;                 // absolute position of the tile's first row
  // two groups in one tile: the union of their key ranges streams through, each row masks to its own
  const int lo_2 = max(0, g.lo + z * g.grow + g.pshift);          // second group's first key (pshift > 0)
  int k_begin = lo_z, k_end = hi_z + g.pshift;
  if (g.window) k_begin = max(k_begin, qpos0 - g.window + 1);
  if (g.causal) k_end = min(k_end, qpos0 + rows_here - 1 - g.causal_excl + 1);
  const int n_tiles = k_end > k_begin ? (k_end - k_begin + KT - 1) / KT : 0;

  if (threadIdx.x == 0) {
    *serr = 0;
    mbar_init(qfull, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(kfull(s), 1);
      mbar_init(vfull(s), 1);
      mbar_init(kvempty(s), 1);
      mbar_init(pvfull(s), 1);
      mbar_init(pvfree(s), 4);
    }
    mbar_init(sfull, 1);
    mbar_init(sfree, 4);
    mbar_init(pfull, 4);
    fence_barrier_init();
  }
  if (warp == 1) tmem_alloc(tmem_slot, C::TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t sQ = base + C::q_off, sK = base + C::k_off, sV = base + C::v_off, sP = base + C::p_off;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0 && n_tiles > 0) {
      mbar_expect_tx(qfull, C::Q_BYTES);
#pragma unroll
      for (int sl = 0; sl < DH / 64; ++sl)
#pragma unroll
        for (int rb = 0; rb < BM / 64; ++rb)
          tma_load_3d(sQ + sl * (BM * 128) + rb * 8192, &tmQ, qfull, h * DH + 64 * sl, z * g.grow + row0 + 64 * rb, b);
      int t = 0;
      for (; t < n_tiles; ++t) {
        const int s = t & 1, k0 = k_begin + t * KT;
        if (!mbar_wait(kvempty(s), ((t >> 1) & 1) ^ 1, serr)) break;
        mbar_expect_tx(kfull(s), C::KV_BYTES);
#pragma unroll
        for (int sl = 0; sl < DH / 64; ++sl)
#pragma unroll
          for (int rb = 0; rb < 2; ++rb)
            tma_load_3d(sK + s * C::KV_BYTES + sl * (KT * 128) + rb * 8192, &tmK, kfull(s), h * DH + 64 * sl, k0 + 64 * rb, b);
        mbar_expect_tx(vfull(s), C::KV_BYTES);
#pragma unroll
        for (int kb = 0; kb < 2; ++kb)
#pragma unroll
          for (int nb = 0; nb < DH / 64; ++nb)
            tma_load_3d(sV + s * C::KV_BYTES + (kb * (DH / 64) + nb) * 8192, &tmV, vfull(s), h * DH + 64 * nb, k0 + 64 * kb, b);
      }
      if (*serr) {
        // another role gave up: nobody will consume the tiles in flight; let them land before the CTA ends
        volatile int ignore = 0;
        for (int u = max(0, t - 2); u < t; ++u) {
          mbar_wait(kfull(u & 1), (u >> 1) & 1, &ignore);
          mbar_wait(vfull(u & 1), (u >> 1) & 1, &ignore);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0 && n_tiles > 0) {
      constexpr uint32_t idS = instr_desc(BM, KT, 0, 0), idPV = instr_desc(BM, DH, 0, 1);
      const uint32_t tS = tmem_base, tPV = tmem_base + KT;
      auto issue_S = [&](int s) {
#pragma unroll
        for (int k = 0; k < DH / 16; ++k) {
          const uint64_t da = make_desc(sQ + (k / 4) * (BM * 128) + (k % 4) * 32, 16, 1024);
          const uint64_t db = make_desc(sK + s * C::KV_BYTES + (k / 4) * (KT * 128) + (k % 4) * 32, 16, 1024);
          umma_bf16(tS, da, db, idS, k != 0);
        }
        umma_commit(sfull);
      };
      bool alive = mbar_wait(qfull, 0, serr) && mbar_wait(kfull(0), 0, serr);
      if (alive) {
        tc_fence_after();
        issue_S(0);
      }
      for (int t = 0; t < n_tiles && alive; ++t) {
        const int s = t & 1;
        if (!mbar_wait(pfull, t & 1, serr) || !mbar_wait(vfull(s), (t >> 1) & 1, serr)) break;
        if (t >= 2 && !mbar_wait(pvfree(s), ((t >> 1) - 1) & 1, serr)) break;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < KT / 16; ++kk) {
          const uint64_t da = make_desc(sP + (kk / 4) * (BM * 128) + (kk % 4) * 32, 16, 1024);
          const uint64_t db = make_desc(sV + s * C::KV_BYTES + (kk / 4) * (DH / 64) * 8192 + (kk % 4) * 2048, 8192, 1024);
          umma_bf16(tPV + s * DH, da, db, idPV, kk != 0);
        }
        umma_commit(pvfull(s));
        umma_commit(kvempty(s));           // K_t, V_t and P_t have been read once these products are done
        if (t + 1 < n_tiles) {
          if (!mbar_wait(kfull(s ^ 1), ((t + 1) >> 1) & 1, serr) || !mbar_wait(sfree, t & 1, serr)) break;
          tc_fence_after();
          issue_S(s ^ 1);
        }
      }
    }
  } else {
    // ---------------- softmax / output: one query row per thread ----------------
    const int q = warp & 3;                                  // the TMEM lane quarter this warp may read
    const uint32_t tlane = tmem_base + ((uint32_t)(q * 32) << 16);
    if constexpr (BM == 64) {
      // M = 64: the accumulator's rows 16q .. 16q+15 sit in lanes 0..15 of quarter q.  They are read with the
      // 16-lane x 256-bit shape, which hands every thread of the warp the accumulator fragment of a warp-level
      // MMA: thread t owns rows rA = 16q + t/4 and rB = rA + 8, columns 8j + 2(t%4), +1 of every 8-column
      // group j.  All 32 lanes work; row maxima are reduced over the 4 threads of a quad, the running sum
      // stays a per-thread partial until the end, and P goes to shared memory with stmatrix (the fragment is
      // its register layout; one 16-byte row per 8-column group, at its swizzled place).
      const int t4 = lane & 3, rA = q * 16 + (lane >> 2), rB = rA + 8;
      int jloA = lo_z, jhiA = hi_z, jloB = lo_z, jhiB = hi_z;
      if (g.window) { jloA = max(jloA, qpos0 + rA - g.window + 1); jloB = max(jloB, qpos0 + rB - g.window + 1); }
      if (g.causal) { jhiA = min(jhiA, qpos0 + rA - g.causal_excl + 1); jhiB = min(jhiB, qpos0 + rB - g.causal_excl + 1); }
      float mA = -INFINITY, mB = -INFINITY, lA = 0.f, lB = 0.f, aprevA = 1.f, aprevB = 1.f;
      float OA[DH / 4], OB[DH / 4];                          // this thread's pairs of both rows
#pragma unroll
      for (int i = 0; i < DH / 4; ++i) OA[i] = OB[i] = 0.f;
      // stmatrix row address of this thread: matrix lane/8 of each x4 store, row lane%8
      const int smat = lane >> 3, srow = q * 16 + (smat & 1) * 8 + (lane & 7);
      bool alive = n_tiles > 0;
      auto wwait = [&](uint32_t bar, uint32_t parity) { return __all_sync(0xffffffffu, mbar_wait(bar, parity, serr)); };
      auto fold = [&](int u, float alA, float alB) {         // O = O * alpha + (P V) of tile u
        const int s = u & 1;
        if (!wwait(pvfull(s), (u >> 1) & 1)) return false;
        tc_fence_after();
#pragma unroll
        for (int c0 = 0; c0 < DH; c0 += 64) {
          uint32_t r[32];
          tmem_ld_16x256b_x8(tlane + KT + s * DH + c0, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int o = (c0 >> 2) + 2 * j;
            OA[o] = OA[o] * alA + __uint_as_float(r[4 * j]);
            OA[o + 1] = OA[o + 1] * alA + __uint_as_float(r[4 * j + 1]);
            OB[o] = OB[o] * alB + __uint_as_float(r[4 * j + 2]);
            OB[o + 1] = OB[o + 1] * alB + __uint_as_float(r[4 * j + 3]);
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(pvfree(s));
        return true;
      };
      for (int t = 0; t < n_tiles && alive; ++t) {
        const int k0 = k_begin + t * KT;
        if (!wwait(sfull, t & 1)) { alive = false; break; }
        tc_fence_after();
        const bool mask = (k0 + KT > k_end) || (g.causal && k0 + KT - 1 > qpos0 - g.causal_excl) ||
                          (g.window && k0 < qpos0 + rows_here - 1 - g.window + 1);
        uint32_t r[64];
        tmem_ld_16x256b_x16(tlane, r);
        tmem_ld_wait();
        // S is in registers: the next tile's scores may be issued
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(sfree);
        float mxA = -INFINITY, mxB = -INFINITY;
        if (mask) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const int kj = k0 + 8 * j + 2 * t4 + e;
              if (!(kj >= jloA && kj < jhiA)) r[4 * j + e] = 0xff800000u;          // -inf
              if (!(kj >= jloB && kj < jhiB)) r[4 * j + 2 + e] = 0xff800000u;
            }
          }
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          mxA = fmaxf(mxA, fmaxf(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1])));
          mxB = fmaxf(mxB, fmaxf(__uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3])));
        }
        mxA = quad_max(mxA);
        mxB = quad_max(mxB);
        const float mnA = fmaxf(mA, mxA * g.scale_log2), mnB = fmaxf(mB, mxB * g.scale_log2);
        const float subA = mnA == -INFINITY ? 0.f : mnA, subB = mnB == -INFINITY ? 0.f : mnB;
        const float alA = exp2f(mA - subA), alB = exp2f(mB - subB);
        mA = mnA;
        mB = mnB;
        // P of tile t-1 must have been read by its product before P of tile t overwrites it
        if (t >= 1 && !fold(t - 1, aprevA, aprevB)) { alive = false; break; }
        float sumA = 0.f, sumB = 0.f;
#pragma unroll
        for (int n = 0; n < 8; ++n) {                         // 16 keys per stmatrix.x4
          uint32_t pk[4];
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            const int j = 2 * n + u;
            const float a0 = exp2f(fmaf(__uint_as_float(r[4 * j]), g.scale_log2, -subA));      // exp2(-inf) = 0
            const float a1 = exp2f(fmaf(__uint_as_float(r[4 * j + 1]), g.scale_log2, -subA));
            const float b0 = exp2f(fmaf(__uint_as_float(r[4 * j + 2]), g.scale_log2, -subB));
            const float b1 = exp2f(fmaf(__uint_as_float(r[4 * j + 3]), g.scale_log2, -subB));
            sumA += a0 + a1;
            sumB += b0 + b1;
            pk[2 * u] = pack_bf16(a0, a1);                   // matrix 2u: rows rA.., key group j
            pk[2 * u + 1] = pack_bf16(b0, b1);               // matrix 2u+1: rows rB.., key group j
          }
          const int jg = 2 * n + (smat >> 1);                 // the 8-key group whose row this thread addresses
          stsm_x4(sP + (jg >> 3) * (BM * 128) + srow * 128 + (((jg & 7) ^ (srow & 7)) << 4), pk[0], pk[1], pk[2], pk[3]);
        }
        lA = lA * alA + sumA;
        lB = lB * alB + sumB;
        aprevA = alA;
        aprevB = alB;
        fence_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(pfull);
      }
      if (alive && n_tiles > 0) alive = fold(n_tiles - 1, aprevA, aprevB);
      lA = quad_sum(lA);
      lB = quad_sum(lB);
      if (alive || n_tiles == 0) {
        const int G_ = (int)(gridDim.z / g.tiles_q);
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int row = half ? rB : rA;
          if (row >= rows_here) continue;
          const float l = half ? lB : lA, m = half ? mB : mA;
          const float* O = half ? OB : OA;
          const float inv = l > 0.f ? 1.f / l : 0.f;
          const long long orow = ((long long)((b * G_ + z) * g.Lq + row0 + row) * g.H + h);
          const float ln = l > 0.f ? (m + log2f(l)) * 0.6931471805599453f : DMB_NEG;
          if (g.mf_o) {                                      // fp32 outputs: the merged partial
            const long long wrow = (long long)z * g.Lq + row0 + row;          // row of the launch's window
            const float* of = g.mf_o + b * g.mf_bs_vec + (wrow * g.H + h) * DH;
            float wf, wn;
            const float lc = merge_weights(g.mf_lse[b * g.mf_bs_sca + wrow * g.H + h], ln, wf, wn);
#pragma unroll
            for (int j = 0; j < DH / 8; ++j) {
              const int d = 8 * j + 2 * t4;
              const float2 f2 = *reinterpret_cast<const float2*>(of + d);
              const float2 n2 = make_float2(O[2 * j] * inv, O[2 * j + 1] * inv);
              *reinterpret_cast<float2*>(reinterpret_cast<float*>(o_out) + orow * DH + d) =
                  make_float2(wf * f2.x + wn * n2.x, wf * f2.y + wn * n2.y);
              if (g.m_on) *reinterpret_cast<float2*>(g.m_on + orow * DH + d) = n2;
            }
            if (t4 == 0) {
              lse_out[orow] = lc;
              g.m_wf[orow] = wf;
              g.m_wn[orow] = wn;
              if (g.m_lsen) g.m_lsen[orow] = ln;
            }
            continue;
          }
#pragma unroll
          for (int j = 0; j < DH / 8; ++j) {
            const int d = 8 * j + 2 * t4;
            if (g.o_bf16)
              *reinterpret_cast<uint32_t*>(reinterpret_cast<bf16*>(o_out) + orow * DH + d) =
                  pack_bf16(O[2 * j] * inv, O[2 * j + 1] * inv);
            else
              *reinterpret_cast<float2*>(reinterpret_cast<float*>(o_out) + orow * DH + d) =
                  make_float2(O[2 * j] * inv, O[2 * j + 1] * inv);
          }
          if (t4 == 0) lse_out[orow] = ln;
        }
      }
    } else {
    const int row = q * 32 + lane;
    const bool has_row = true;
    const int qpos = qpos0 + row;
    const bool second = g.pshift && row >= 64;
    int jlo = second ? lo_2 : lo_z, jhi = hi_z + (second ? g.pshift : 0);   // allowed keys of this row: jlo <= j < jhi
    if (g.window) jlo = max(jlo, qpos - g.window + 1);
    if (g.causal) jhi = min(jhi, qpos - g.causal_excl + 1);
    float m = -INFINITY, l = 0.f, alpha_prev = 1.f;
    float O[DH];
#pragma unroll
    for (int d = 0; d < DH; ++d) O[d] = 0.f;
    uint8_t* pP = base_ptr + C::p_off;
    bool alive = n_tiles > 0;
    auto wwait = [&](uint32_t bar, uint32_t parity) { return __all_sync(0xffffffffu, mbar_wait(bar, parity, serr)); };
    auto fold = [&](int u, float alpha) {                    // O = O * alpha + (P V) of tile u
      const int s = u & 1;
      if (!wwait(pvfull(s), (u >> 1) & 1)) return false;
      tc_fence_after();
#pragma unroll
      for (int c0 = 0; c0 < DH; c0 += 64) {
        uint32_t r[64];
        tmem_ld32(tlane + KT + s * DH + c0, *reinterpret_cast<uint32_t (*)[32]>(&r[0]));
        tmem_ld32(tlane + KT + s * DH + c0 + 32, *reinterpret_cast<uint32_t (*)[32]>(&r[32]));
        tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < 64; ++e) O[c0 + e] = O[c0 + e] * alpha + __uint_as_float(r[e]);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(pvfree(s));
      return true;
    };
    for (int t = 0; t < n_tiles && alive; ++t) {
      const int k0 = k_begin + t * KT;
      if (!wwait(sfull, t & 1)) { alive = false; break; }
      tc_fence_after();
      // a tile needs per-element masks only where it crosses a row's range
      const bool mask = (k0 + KT > k_end) || (k0 < lo_z) || (g.causal && k0 + KT - 1 > qpos0 - g.causal_excl) ||
                        (g.window && k0 < qpos0 + rows_here - 1 - g.window + 1) ||
                        (g.pshift && (k0 + KT > hi_z || k0 < lo_2));
      float mx = -INFINITY;
#pragma unroll 1
      for (int c0 = 0; c0 < KT; c0 += 64) {                 // two loads in flight per wait
        uint32_t r[64];
        tmem_ld32(tlane + c0, *reinterpret_cast<uint32_t (*)[32]>(&r[0]));
        tmem_ld32(tlane + c0 + 32, *reinterpret_cast<uint32_t (*)[32]>(&r[32]));
        tmem_ld_wait();
        if (mask) {
#pragma unroll
          for (int e = 0; e < 64; ++e) {
            const int j = k0 + c0 + e;
            mx = fmaxf(mx, (j >= jlo && j < jhi) ? __uint_as_float(r[e]) : -INFINITY);
          }
        } else {
#pragma unroll
          for (int e = 0; e < 64; ++e) mx = fmaxf(mx, __uint_as_float(r[e]));
        }
      }
      const float m_new = fmaxf(m, mx * g.scale_log2);
      const float sub = m_new == -INFINITY ? 0.f : m_new;
      const float alpha = exp2f(m - sub);                    // exp2(-inf) = 0 on a row's first live tile
      m = m_new;
      float sum = 0.f;
      // the P V product of tile t-2 used this P buffer's neighbours only; P itself is free once P V of tile
      // t-1 has been issued AND read its operands, which kvempty / pvfull of t-1 imply; wait for pvfull(t-1)
      // by folding tile t-1 first
      if (t >= 1) {
        if (!fold(t - 1, alpha_prev)) { alive = false; break; }
      }
#pragma unroll 1
      for (int c0 = 0; c0 < KT; c0 += 64) {                 // one 64-key slab of P per round
        uint32_t r[64];
        tmem_ld32(tlane + c0, *reinterpret_cast<uint32_t (*)[32]>(&r[0]));
        tmem_ld32(tlane + c0 + 32, *reinterpret_cast<uint32_t (*)[32]>(&r[32]));
        tmem_ld_wait();
        uint32_t pk[32];
#pragma unroll
        for (int e = 0; e < 64; e += 2) {
          const int j = k0 + c0 + e;
          float p0 = exp2f(fmaf(__uint_as_float(r[e]), g.scale_log2, -sub));
          float p1 = exp2f(fmaf(__uint_as_float(r[e + 1]), g.scale_log2, -sub));
          if (mask) {
            if (!(j >= jlo && j < jhi)) p0 = 0.f;
            if (!(j + 1 >= jlo && j + 1 < jhi)) p1 = 0.f;
          }
          sum += p0 + p1;
          pk[e >> 1] = pack_bf16(p0, p1);
        }
        if (has_row) {
          // operand layout of P (K-major, 128-byte swizzle): 64-key slab, row pitch 128 B, 16-byte chunk c of
          // row r stored at chunk c ^ (r & 7)
          uint8_t* rowp = pP + (c0 >> 6) * (BM * 128) + row * 128;
#pragma unroll
          for (int c = 0; c < 8; ++c)
            *reinterpret_cast<uint4*>(rowp + ((c ^ (row & 7)) << 4)) =
                make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
        }
      }
      l = l * alpha + sum;
      alpha_prev = alpha;
      // S has been read twice and P is in shared memory: release S, publish P
      tc_fence_before();
      fence_async_smem();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(sfree);
        mbar_arrive(pfull);
      }
    }
    if (alive && n_tiles > 0) alive = fold(n_tiles - 1, alpha_prev);
    // ---- write the row ----
    if (has_row && row < rows_here && (alive || n_tiles == 0)) {
      const float inv = l > 0.f ? 1.f / l : 0.f;
      const long long orow = ((long long)((b * (int)(gridDim.z / g.tiles_q) + z) * g.Lq + row0 + row) * g.H + h);
      const float ln = l > 0.f ? (m + log2f(l)) * 0.6931471805599453f : DMB_NEG;
      if (g.mf_o) {                                          // fp32 outputs: the merged partial
        const long long wrow = (long long)z * g.Lq + row0 + row;
        const float* of = g.mf_o + b * g.mf_bs_vec + (wrow * g.H + h) * DH;
        float wf, wn;
        const float lc = merge_weights(g.mf_lse[b * g.mf_bs_sca + wrow * g.H + h], ln, wf, wn);
        float* dst = reinterpret_cast<float*>(o_out) + orow * DH;
#pragma unroll
        for (int d = 0; d < DH; d += 4) {
          const float4 f4 = *reinterpret_cast<const float4*>(of + d);
          const float4 n4 = make_float4(O[d] * inv, O[d + 1] * inv, O[d + 2] * inv, O[d + 3] * inv);
          *reinterpret_cast<float4*>(dst + d) =
              make_float4(wf * f4.x + wn * n4.x, wf * f4.y + wn * n4.y, wf * f4.z + wn * n4.z, wf * f4.w + wn * n4.w);
          if (g.m_on) *reinterpret_cast<float4*>(g.m_on + orow * DH + d) = n4;
        }
        lse_out[orow] = lc;
        g.m_wf[orow] = wf;
        g.m_wn[orow] = wn;
        if (g.m_lsen) g.m_lsen[orow] = ln;
      } else if (g.o_bf16) {
        bf16* dst = reinterpret_cast<bf16*>(o_out) + orow * DH;
#pragma unroll
        for (int d = 0; d < DH; d += 8)
          *reinterpret_cast<uint4*>(dst + d) =
              make_uint4(pack_bf16(O[d] * inv, O[d + 1] * inv), pack_bf16(O[d + 2] * inv, O[d + 3] * inv),
                         pack_bf16(O[d + 4] * inv, O[d + 5] * inv), pack_bf16(O[d + 6] * inv, O[d + 7] * inv));
      } else {
        float* dst = reinterpret_cast<float*>(o_out) + orow * DH;
#pragma unroll
        for (int d = 0; d < DH; d += 4)
          *reinterpret_cast<float4*>(dst + d) = make_float4(O[d] * inv, O[d + 1] * inv, O[d + 2] * inv, O[d + 3] * inv);
      }
      if (!g.mf_o) lse_out[orow] = ln;
    }
    }   // BM == 128
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
  if (threadIdx.x == 0 && *serr) atomicExch(gerr, 1);
}

template <int DH, int BM>
int launch(const void* q, TView vq, int q_rows, const void* Kc, const void* Vc, TView vc, int tape_rows, void* o,
           float* lse, int B, int G, const Geo& g, int* gerr, cudaStream_t st) {
  using C = Cfg<DH, BM>;
  auto kern = attn_fwd_tc_kernel<DH, BM>;
  static bool configured = false;
  const int smem = C::total;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  CUtensorMap tq, tk, tv;
  const long long cols = (long long)g.H * DH;
  int rc;
  if ((rc = make_map_3d(&tq, q, cols, q_rows, B, vq.rs, B > 1 ? vq.bs : (long long)q_rows * vq.rs, 64, 64))) return rc;
  // rows at and beyond the end of the largest key range are outside the map: the copy engine zero-fills them
  // (an empty range for every group still needs a valid map: one row, never loaded)
  const int k_rows = max(1, min(tape_rows, g.hi + (G - 1) * g.grow + g.pshift));
  const long long kbs = B > 1 ? vc.bs : (long long)tape_rows * vc.rs;
  if ((rc = make_map_3d(&tk, Kc, cols, k_rows, B, vc.rs, kbs, 64, 64))) return rc;
  if ((rc = make_map_3d(&tv, Vc, cols, k_rows, B, vc.rs, kbs, 64, 64))) return rc;
  kern<<<dim3(g.H, B, G * g.tiles_q), NTHREADS, smem, st>>>(tq, tk, tv, o, lse, g, gerr);
  DMB_CHECK_LAUNCH();
  return 0;
}

}  // namespace

extern "C" {

// Attention forward of query rows against tape rows, on tcgen05.
//   q            bf16 view (batch stride vq.bs, row stride vq.rs elements, heads x DH dense in a row) with
//                q_rows rows per batch; group z uses rows [z*grow, z*grow + Lq)
//   Kc, Vc       bf16 tapes [B, tape_rows, H, DH] with strides vc
//   o, lse       dense [B, G, Lq, H, DH] (fp32, or bf16 when o_bf16) and [B, G, Lq, H] fp32
//   keys of group z: max(0, lo + z*grow) <= j < hi + z*grow; query row i sits at qbase + z*grow + i;
//   causal: j <= position - causal_excl; window > 0: j > position - window
//   bm: 64 or 128 query rows per CTA.  gerr: device int, set to 1 if a pipeline wait ran out.
//   mf_o, mf_lse (optional): another partial of the same rows (fp32, rows by absolute position from the launch's
//   first row, batch strides mf_bs_vec / mf_bs_sca); the outputs o / lse are then the MERGED partial, m_wf / m_wn
//   [B, G, Lq, H] receive the two weights and m_on / m_lsen (optional, dense like o / lse) this read's own partial.
// Requirements: 16-byte aligned pointers, strides multiples of 8 elements, dh 64 or 128.
int dmb_attn_fwd_tc_merged(const void* q, TView vq, int q_rows, const void* Kc, const void* Vc, TView vc, int tape_rows,
                           void* o, int o_bf16, float* lse, int B, int G, int Lq, int H, int dh, int lo, int hi,
                           int qbase, int grow, float scale, int window, int causal, int causal_excl, int bm,
                           int pair_shift, const float* mf_o, const float* mf_lse, long long mf_bs_vec,
                           long long mf_bs_sca, float* m_wf, float* m_wn, float* m_on, float* m_lsen, int* gerr,
                           cudaStream_t st) {
  if (!encode_fn()) return -10;
  if ((dh != 64 && dh != 128) || (bm != 64 && bm != 128) || Lq <= 0 || B <= 0 || G <= 0) return -1;
  // pair_shift > 0: a "group" is two 64-row groups of one 128-row tile whose key ranges differ by pair_shift rows
  if (pair_shift && (bm != 128 || Lq != 128 || causal)) return -1;
  // merged outputs are fp32 and need both weight arrays
  if (mf_o && (o_bf16 || !mf_lse || !m_wf || !m_wn || (m_on != nullptr) != (m_lsen != nullptr))) return -1;
  Geo g = {};
  g.pshift = pair_shift;
  g.mf_o = mf_o; g.mf_lse = mf_lse; g.mf_bs_vec = mf_bs_vec; g.mf_bs_sca = mf_bs_sca;
  g.m_wf = m_wf; g.m_wn = m_wn; g.m_on = m_on; g.m_lsen = m_lsen;
  g.H = H; g.Lq = Lq; g.lo = lo; g.hi = hi; g.qbase = qbase; g.grow = grow; g.window = window;
  g.causal = causal; g.causal_excl = causal_excl; g.tiles_q = (Lq + bm - 1) / bm;
  g.o_bf16 = o_bf16; g.scale_log2 = scale * 1.4426950408889634f;
  if (dh == 64) {
    if (bm == 64) return launch<64, 64>(q, vq, q_rows, Kc, Vc, vc, tape_rows, o, lse, B, G, g, gerr, st);
    return launch<64, 128>(q, vq, q_rows, Kc, Vc, vc, tape_rows, o, lse, B, G, g, gerr, st);
  }
  if (bm == 64) return launch<128, 64>(q, vq, q_rows, Kc, Vc, vc, tape_rows, o, lse, B, G, g, gerr, st);
  return launch<128, 128>(q, vq, q_rows, Kc, Vc, vc, tape_rows, o, lse, B, G, g, gerr, st);
}

// the plain read (no merge)
int dmb_attn_fwd_tc(const void* q, TView vq, int q_rows, const void* Kc, const void* Vc, TView vc, int tape_rows,
                    void* o, int o_bf16, float* lse, int B, int G, int Lq, int H, int dh, int lo, int hi, int qbase,
                    int grow, float scale, int window, int causal, int causal_excl, int bm, int pair_shift,
                    int* gerr, cudaStream_t st) {
  return dmb_attn_fwd_tc_merged(q, vq, q_rows, Kc, Vc, vc, tape_rows, o, o_bf16, lse, B, G, Lq, H, dh, lo, hi, qbase, grow,
                                scale, window, causal, causal_excl, bm, pair_shift, nullptr, nullptr, 0, 0, nullptr,
                                nullptr, nullptr, nullptr, gerr, st);
}

}  // extern "C"

// =================================================================================================
// Backward of a read of the tape, on tcgen05: both sides of the owner-computes scheme in one kernel.
//
//   query side (KEYSIDE = 0): the CTA owns 64 query rows (Q, d o) and streams key tiles K_t, V_t;
//       S = Q K_t^T, dP = d o V_t^T, dS = exp(S - lse) (dP - corr) scale  (lse, corr per ROW),
//       dQ += dS K_t                                   accumulated in tensor memory over all tiles
//   key side   (KEYSIDE = 1): the CTA owns the 64 tape rows of a chunk (K, V) and streams tiles of the
//       LATER query rows Q_t, d o_t of the sequence (every one of them read this chunk);
//       S^T = K Q_t^T, dP^T = V d o_t^T, P^T = exp(S^T - lse), dS^T = P^T (dP^T - corr) scale
//       (lse, corr per COLUMN, staged in shared memory), dK += dS^T Q_t, dV += P^T d o_t.
//
// corr = d o . o - d lse of the read.  The streamed tile serves twice from one shared-memory copy: K-major
// as the B operand of the score products and, through a descriptor that walks its rows, as the
// row-major B operand of the gradient products.  M = 64 products: the accumulator's 64 rows sit in lanes
// 0..15 of each 32-lane quarter and are read as warp-MMA fragments (16-lane x 256-bit tcgen05.ld), dS and
// P go back to shared memory with stmatrix.  Tensor memory: S 64 | dP 64 | accumulators: 256 columns at head dim 64 (two CTAs
// per SM), 512 at head dim 128 on the key side.
namespace {

constexpr int BT = 64;                  // owner rows and streamed rows per tile

template <int DH, int KEYSIDE>
struct BCfg {
  static constexpr int T_BYTES = BT * DH * 2;            // one 64-row tile
  static constexpr int a_off = 0;                        // owner tiles A1 (Q | K), A2 (d o | V)
  static constexpr int y_off = 2 * T_BYTES;              // streamed pairs (Y1, Y2), two stages
  static constexpr int ds_off = y_off + 4 * T_BYTES;     // dS (and P on the key side), 8 KB each
  static constexpr int sc_off = ds_off + 2 * BT * 128;   // per-column lse / corr: [math warp][stage][2][64] floats
  static constexpr int bar_off = sc_off + 4096;
  static constexpr int total = bar_off + 256;
  static constexpr int ACC = KEYSIDE ? 2 * DH : DH;
  static constexpr int TMEM_COLS = 128 + ACC <= 256 ? 256 : 512;
};

struct BGeo {
  int H, T, C, lo, hi, qbase, grow, window, span, accumulate, q_start, q_end;
  long long o_bs, o_rs;          // output view: element (b, row, col) at b * o_bs + row * o_rs + col; group z at rows z * 64
  float scale, scale_log2;
};

template <int DH, int KEYSIDE>
__global__ void __launch_bounds__(NTHREADS, (BCfg<DH, KEYSIDE>::TMEM_COLS == 256 ? 2 : 1)) attn_bwd_tc_kernel(
    const __grid_constant__ CUtensorMap tmA1, const __grid_constant__ CUtensorMap tmA2,
    const __grid_constant__ CUtensorMap tmY1, const __grid_constant__ CUtensorMap tmY2,
    const float* __restrict__ lse, const float* __restrict__ corr, float* __restrict__ out1,
    float* __restrict__ out2, const BGeo g, int* __restrict__ gerr) {
  using C = BCfg<DH, KEYSIDE>;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t base = smem_u32(smem_raw);
  if (base & 1023u) {
    if (threadIdx.x == 0) atomicExch(gerr, 2);
    return;
  }
  uint8_t* base_ptr = smem_raw;
  const uint32_t bar0 = base + C::bar_off;
  // barriers: afull, yfull[2], yempty[2], sdfull, sdfree, dsfull, dsfree, accdone
  const uint32_t afull = bar0;
  auto yfull = [&](int s) { return bar0 + 8u * (1 + s); };
  auto yempty = [&](int s) { return bar0 + 8u * (3 + s); };
  const uint32_t sdfull = bar0 + 8u * 5, sdfree = bar0 + 8u * 6, dsfull = bar0 + 8u * 7, dsfree = bar0 + 8u * 8,
                 accdone = bar0 + 8u * 9;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(base_ptr + C::bar_off + 8 * 10);
  volatile int* serr = reinterpret_cast<volatile int*>(base_ptr + C::bar_off + 8 * 11);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.x, b = blockIdx.y, z = blockIdx.z, G = gridDim.z;
  // owner rows and the streamed range [s_begin, s_end) (tape rows on the query side, query positions on the
  // key side); own_pos: absolute position of owner row 0
  int own_row0, own_pos, s_begin, s_end;
  if (!KEYSIDE) {
    own_row0 = z * g.grow;                                // row of the q / d o views
    own_pos = g.qbase + z * g.grow;
    s_begin = max(0, g.lo + z * g.grow);
    s_end = g.hi + z * g.grow;
    if (g.window) s_begin = min(s_end, max(s_begin, own_pos - g.window + 1));
  } else {
    own_row0 = own_pos = g.lo + z * g.grow;               // tape rows of the chunk (lo = first chunk's row 0)
    s_begin = max(g.q_start, own_pos + g.C);
    s_end = min(g.q_end, own_pos + g.span);
    if (g.window) s_end = min(s_end, own_pos + BT - 1 + g.window);   // later rows cannot see any owner key
  }
  const int n_tiles = s_end > s_begin ? (s_end - s_begin + BT - 1) / BT : 0;

  if (threadIdx.x == 0) {
    *serr = 0;
    mbar_init(afull, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(yfull(s), 1);
      mbar_init(yempty(s), 1);
    }
    mbar_init(sdfull, 1);
    mbar_init(sdfree, 4);
    mbar_init(dsfull, 4);
    mbar_init(dsfree, 1);
    mbar_init(accdone, 1);
    fence_barrier_init();
  }
  if (warp == 1) tmem_alloc(tmem_slot, C::TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t sA1 = base + C::a_off, sA2 = sA1 + C::T_BYTES, sY = base + C::y_off, sdS = base + C::ds_off,
                 sPm = sdS + BT * 128;
  const uint32_t tS = tmem_base, tdP = tmem_base + 64, tAcc1 = tmem_base + 128, tAcc2 = tmem_base + 128 + DH;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0 && n_tiles > 0) {
      mbar_expect_tx(afull, 2 * C::T_BYTES);
#pragma unroll
      for (int sl = 0; sl < DH / 64; ++sl) {
        tma_load_3d(sA1 + sl * 8192, &tmA1, afull, h * DH + 64 * sl, own_row0, b);
        tma_load_3d(sA2 + sl * 8192, &tmA2, afull, h * DH + 64 * sl, own_row0, b);
      }
      int t = 0;
      for (; t < n_tiles; ++t) {
        const int s = t & 1, r0 = s_begin + t * BT;
        if (!mbar_wait(yempty(s), ((t >> 1) & 1) ^ 1, serr)) break;
        mbar_expect_tx(yfull(s), 2 * C::T_BYTES);
#pragma unroll
        for (int sl = 0; sl < DH / 64; ++sl) {
          tma_load_3d(sY + (2 * s) * C::T_BYTES + sl * 8192, &tmY1, yfull(s), h * DH + 64 * sl, r0, b);
          tma_load_3d(sY + (2 * s + 1) * C::T_BYTES + sl * 8192, &tmY2, yfull(s), h * DH + 64 * sl, r0, b);
        }
      }
      if (*serr) {
        volatile int ignore = 0;
        for (int u = max(0, t - 2); u < t; ++u) mbar_wait(yfull(u & 1), (u >> 1) & 1, &ignore);
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0 && n_tiles > 0) {
      constexpr uint32_t idS = instr_desc(BT, BT, 0, 0), idG = instr_desc(BT, DH, 0, 1);
      auto issue_scores = [&](int s) {                      // S = A1 Y1^T, dP = A2 Y2^T
        const uint32_t y1 = sY + (2 * s) * C::T_BYTES, y2 = y1 + C::T_BYTES;
#pragma unroll
        for (int k = 0; k < DH / 16; ++k) {
          const uint32_t o = (k / 4) * 8192 + (k % 4) * 32;
          umma_bf16(tS, make_desc(sA1 + o, 16, 1024), make_desc(y1 + o, 16, 1024), idS, k != 0);
        }
#pragma unroll
        for (int k = 0; k < DH / 16; ++k) {
          const uint32_t o = (k / 4) * 8192 + (k % 4) * 32;
          umma_bf16(tdP, make_desc(sA2 + o, 16, 1024), make_desc(y2 + o, 16, 1024), idS, k != 0);
        }
        umma_commit(sdfull);
      };
      auto issue_grads = [&](int u) {                       // acc1 += dS Y1 (and acc2 += P Y2) of tile u
        const int s = u & 1;
        const uint32_t y1 = sY + (2 * s) * C::T_BYTES, y2 = y1 + C::T_BYTES;
#pragma unroll
        for (int kk = 0; kk < BT / 16; ++kk)
          umma_bf16(tAcc1, make_desc(sdS + kk * 32, 16, 1024), make_desc(y1 + kk * 2048, 8192, 1024), idG,
                    (u | kk) != 0);
        if (KEYSIDE) {
#pragma unroll
          for (int kk = 0; kk < BT / 16; ++kk)
            umma_bf16(tAcc2, make_desc(sPm + kk * 32, 16, 1024), make_desc(y2 + kk * 2048, 8192, 1024), idG,
                      (u | kk) != 0);
        }
        umma_commit(dsfree);               // dS / P may be overwritten
        umma_commit(yempty(s));            // the streamed pair of tile u has been read by both products
      };
      bool alive = mbar_wait(afull, 0, serr);
      for (int t = 0; t < n_tiles && alive; ++t) {
        const int s = t & 1;
        if (!mbar_wait(yfull(s), (t >> 1) & 1, serr)) { alive = false; break; }
        if (t > 0 && !mbar_wait(sdfree, (t - 1) & 1, serr)) { alive = false; break; }
        tc_fence_after();
        issue_scores(s);
        if (t > 0) {
          if (!mbar_wait(dsfull, (t - 1) & 1, serr)) { alive = false; break; }
          tc_fence_after();
          issue_grads(t - 1);
        }
      }
      if (alive && mbar_wait(dsfull, (n_tiles - 1) & 1, serr)) {
        tc_fence_after();
        issue_grads(n_tiles - 1);
        umma_commit(accdone);
      }
    }
  } else {
    // ---------------- gradient math ----------------
    // The M = 64 accumulators are read as warp-MMA fragments (16-lane x 256-bit loads): thread t of the warp
    // of quarter q owns the owner rows rA = 16q + t/4 and rB = rA + 8 and the streamed columns 8j + 2(t%4), +1.
    const int q = warp & 3, t4 = lane & 3, rA = q * 16 + (lane >> 2), rB = rA + 8;
    const uint32_t tlane = tmem_base + ((uint32_t)(q * 32) << 16);
    auto wwait = [&](uint32_t bar, uint32_t parity) { return __all_sync(0xffffffffu, mbar_wait(bar, parity, serr)); };
    // dense per-row arrays: [B, G, C, H]
    const long long orowA = ((long long)((b * G + z) * g.C + rA) * g.H + h), orowB = orowA + 8ll * g.H;
    float L2A = 0.f, L2B = 0.f, cA = 0.f, cB = 0.f;
    if (!KEYSIDE) {
      L2A = lse[orowA] * 1.4426950408889634f;
      L2B = lse[orowB] * 1.4426950408889634f;
      cA = corr[orowA];
      cB = corr[orowB];
    }
    // every math warp stages its own copy of the per-column scalars, so no barrier spans the warps
    float* sc = reinterpret_cast<float*>(base_ptr + C::sc_off) + q * 256;
    const int smat = lane >> 3, srow = q * 16 + (smat & 1) * 8 + (lane & 7);   // stmatrix row this thread addresses
    bool alive = n_tiles > 0;
    for (int t = 0; t < n_tiles && alive; ++t) {
      const int c0pos = s_begin + t * BT;                    // position / tape row of streamed column 0
      if (KEYSIDE) {
        // stage this tile's per-column lse (log2 domain) and corr: [stage][2][64]; the slot written here
        // was last read two tiles ago by this same warp
#pragma unroll
        for (int i = lane; i < BT; i += 32) {
          const int tpos = c0pos + i;
          float vl = 0.f, vc_ = 0.f;
          if (tpos < s_end) {
            const long long idx = ((long long)b * g.T + tpos) * g.H + h;
            vl = lse[idx] * 1.4426950408889634f;
            vc_ = corr[idx];
          }
          sc[(t & 1) * 128 + i] = vl;
          sc[(t & 1) * 128 + 64 + i] = vc_;
        }
        __syncwarp();
      }
      if (!wwait(sdfull, t & 1)) { alive = false; break; }
      tc_fence_after();
      uint32_t rs[32], rd[32];
      tmem_ld_16x256b_x8(tlane, rs);
      tmem_ld_16x256b_x8(tlane + 64, rd);
      tmem_ld_wait();
      // S and dP are in registers: the next tile's score products may overwrite them
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(sdfree);
      const bool mask = (c0pos + BT > s_end) || g.window != 0;
      const float* scL = sc + (t & 1) * 128;
      uint32_t pds[16], pp[16];                              // [8-column group j][row A, row B]
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int c = 8 * j + 2 * t4;
        float2 L2c = make_float2(0.f, 0.f), ccc = make_float2(0.f, 0.f);
        if (KEYSIDE) {
          L2c = *reinterpret_cast<const float2*>(scL + c);
          ccc = *reinterpret_cast<const float2*>(scL + 64 + c);
        }
        float p[4], w[4];                                    // (A, c), (A, c+1), (B, c), (B, c+1)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int col = e & 1, rowB = e >> 1;
          const float L2 = KEYSIDE ? (col ? L2c.y : L2c.x) : (rowB ? L2B : L2A);
          const float cc = KEYSIDE ? (col ? ccc.y : ccc.x) : (rowB ? cB : cA);
          float pe = exp2f(fmaf(__uint_as_float(rs[4 * j + e]), g.scale_log2, -L2));
          if (mask) {
            const int cpos = c0pos + c + col, rp = own_pos + (rowB ? rB : rA);
            const int key = KEYSIDE ? rp : cpos, qp = KEYSIDE ? cpos : rp;
            if (cpos >= s_end || (g.window && key <= qp - g.window)) pe = 0.f;
          }
          p[e] = pe;
          w[e] = pe * (__uint_as_float(rd[4 * j + e]) - cc) * g.scale;
        }
        pds[2 * j] = pack_bf16(w[0], w[1]);
        pds[2 * j + 1] = pack_bf16(w[2], w[3]);
        if (KEYSIDE) {
          pp[2 * j] = pack_bf16(p[0], p[1]);
          pp[2 * j + 1] = pack_bf16(p[2], p[3]);
        }
      }
      // the gradient products of the previous tile must have read dS (and P) before they are overwritten
      if (t > 0 && !wwait(dsfree, (t - 1) & 1)) { alive = false; break; }
#pragma unroll
      for (int n = 0; n < 4; ++n) {                           // 16 streamed columns per stmatrix.x4
        const int jg = 2 * n + (smat >> 1);
        const uint32_t a = sdS + srow * 128 + (((jg & 7) ^ (srow & 7)) << 4);
        stsm_x4(a, pds[4 * n], pds[4 * n + 1], pds[4 * n + 2], pds[4 * n + 3]);
        if (KEYSIDE) stsm_x4(a + BT * 128, pp[4 * n], pp[4 * n + 1], pp[4 * n + 2], pp[4 * n + 3]);
      }
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(dsfull);
    }
    // ---- the accumulated gradients ----
    if (alive && n_tiles > 0) alive = wwait(accdone, 0);
    if (alive || n_tiles == 0) {
      if (n_tiles > 0) tc_fence_after();
#pragma unroll 1
      for (int a = 0; a < (KEYSIDE ? 2 : 1); ++a) {
        float* dstA = (a == 0 ? out1 : out2) + b * g.o_bs + (long long)(z * BT + rA) * g.o_rs + (long long)h * DH;
        float* dstB = dstA + 8 * g.o_rs;
#pragma unroll 1
        for (int c0 = 0; c0 < DH; c0 += 64) {
          uint32_t r[32];
          if (n_tiles > 0) {
            tmem_ld_16x256b_x8(tlane + 128 + a * DH + c0, r);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int e = 0; e < 32; ++e) r[e] = 0u;
          }
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int d = c0 + 8 * j + 2 * t4;
            float2 vA = make_float2(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]));
            float2 vB = make_float2(__uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
            if (g.accumulate) {
              const float2 oA = *reinterpret_cast<const float2*>(dstA + d), oB = *reinterpret_cast<const float2*>(dstB + d);
              vA.x += oA.x; vA.y += oA.y; vB.x += oB.x; vB.y += oB.y;
            }
            *reinterpret_cast<float2*>(dstA + d) = vA;
            *reinterpret_cast<float2*>(dstB + d) = vB;
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
  if (threadIdx.x == 0 && *serr) atomicExch(gerr, 1);
}

// ---------------------------------------------------------------------------------------------------------
// Key side with 128 reader rows per tile (head dim 64).  The chunk's K and V (64 keys) stay in shared memory; the
// readers' (q, d o) rows stream in tiles of 128.  Scores are formed with the READERS as the M dimension,
//   S = Q_t K^T, dP = dO_t V^T      (M = 128, N = 64: full-rate MMAs, one accumulator row per thread)
// every math thread owns one reader row (its lse and corr are two scalars, no per-column staging), writes its row
// of P and dS (64 keys = one 128-byte swizzled line) into shared memory, and the gradient products read those
// tiles as M-major A operands and the streamed (d o, q) tiles as N-major B operands:
//   dV += P^T dO_t, dK += dS^T Q_t  (M = 64 keys, N = 64, K = 128 readers).
// Half as many trips round the MMA -> tensor-memory load -> exponentials -> shared-memory store -> MMA chain as the
// 64-reader kernel above.  Tensor memory: S 64 | dP 64 | dK 64 | dV 64 columns: two CTAs per SM.
constexpr int QT = 128;

struct KCfg {
  static constexpr int KV_BYTES = BT * 64 * 2;          // the chunk's K (or V): 8 KB
  static constexpr int Y_BYTES = QT * 64 * 2;           // one streamed tile of q (or d o): 16 KB
  static constexpr int a_off = 0;
  static constexpr int y_off = 2 * KV_BYTES;            // (q, d o) x two stages
  static constexpr int ds_off = y_off + 4 * Y_BYTES;    // dS [128 readers][64 keys], then P
  static constexpr int bar_off = ds_off + 2 * QT * 128;
  static constexpr int total = bar_off + 256;
};

__global__ void __launch_bounds__(NTHREADS, 2) attn_dkv128_tc_kernel(
    const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
    const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmDO,
    const float* __restrict__ lse, const float* __restrict__ corr, float* __restrict__ out1,
    float* __restrict__ out2, const BGeo g, int* __restrict__ gerr) {
  using C = KCfg;
  constexpr int DH = 64;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t base = smem_u32(smem_raw);
  if (base & 1023u) {
    if (threadIdx.x == 0) atomicExch(gerr, 2);
    return;
  }
  uint8_t* base_ptr = smem_raw;
  const uint32_t bar0 = base + C::bar_off;
  const uint32_t afull = bar0;
  auto yfull = [&](int s) { return bar0 + 8u * (1 + s); };
  auto yempty = [&](int s) { return bar0 + 8u * (3 + s); };
  const uint32_t sdfull = bar0 + 8u * 5, sdfree = bar0 + 8u * 6, dsfull = bar0 + 8u * 7, dsfree = bar0 + 8u * 8,
                 accdone = bar0 + 8u * 9;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(base_ptr + C::bar_off + 8 * 10);
  volatile int* serr = reinterpret_cast<volatile int*>(base_ptr + C::bar_off + 8 * 11);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.x, b = blockIdx.y, z = blockIdx.z;
  const int own_pos = g.lo + z * g.grow;                  // tape row of the chunk's first key
  const int s_begin = max(g.q_start, own_pos + g.C);
  int s_end = min(g.q_end, own_pos + g.span);
  if (g.window) s_end = min(s_end, own_pos + BT - 1 + g.window);
  const int n_tiles = s_end > s_begin ? (s_end - s_begin + QT - 1) / QT : 0;

  if (threadIdx.x == 0) {
    *serr = 0;
    mbar_init(afull, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(yfull(s), 1);
      mbar_init(yempty(s), 1);
    }
    mbar_init(sdfull, 1);
    mbar_init(sdfree, 4);
    mbar_init(dsfull, 4);
    mbar_init(dsfree, 1);
    mbar_init(accdone, 1);
    fence_barrier_init();
  }
  if (warp == 1) tmem_alloc(tmem_slot, 256);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t sK = base + C::a_off, sV = sK + C::KV_BYTES, sY = base + C::y_off, sdS = base + C::ds_off,
                 sPm = sdS + QT * 128;
  const uint32_t tS = tmem_base, tdP = tmem_base + 64, tdK = tmem_base + 128, tdV = tmem_base + 192;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0 && n_tiles > 0) {
      mbar_expect_tx(afull, 2 * C::KV_BYTES);
      tma_load_3d(sK, &tmK, afull, h * DH, own_pos, b);
      tma_load_3d(sV, &tmV, afull, h * DH, own_pos, b);
      int t = 0;
      for (; t < n_tiles; ++t) {
        const int s = t & 1, r0 = s_begin + t * QT;
        if (!mbar_wait(yempty(s), ((t >> 1) & 1) ^ 1, serr)) break;
        mbar_expect_tx(yfull(s), 2 * C::Y_BYTES);
        tma_load_3d(sY + (2 * s) * C::Y_BYTES, &tmQ, yfull(s), h * DH, r0, b);
        tma_load_3d(sY + (2 * s + 1) * C::Y_BYTES, &tmDO, yfull(s), h * DH, r0, b);
      }
      if (*serr) {
        volatile int ignore = 0;
        for (int u = max(0, t - 2); u < t; ++u) mbar_wait(yfull(u & 1), (u >> 1) & 1, &ignore);
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0 && n_tiles > 0) {
      constexpr uint32_t idS = instr_desc(QT, BT, 0, 0), idG = instr_desc(BT, DH, 1, 1);
      auto issue_scores = [&](int s) {                      // S = Q_t K^T, dP = dO_t V^T
        const uint32_t yq = sY + (2 * s) * C::Y_BYTES, yo = yq + C::Y_BYTES;
#pragma unroll
        for (int k = 0; k < DH / 16; ++k)
          umma_bf16(tS, make_desc(yq + k * 32, 16, 1024), make_desc(sK + k * 32, 16, 1024), idS, k != 0);
#pragma unroll
        for (int k = 0; k < DH / 16; ++k)
          umma_bf16(tdP, make_desc(yo + k * 32, 16, 1024), make_desc(sV + k * 32, 16, 1024), idS, k != 0);
        umma_commit(sdfull);
      };
      auto issue_grads = [&](int u) {                       // dV += P^T dO_t, dK += dS^T Q_t of tile u
        const int s = u & 1;
        const uint32_t yq = sY + (2 * s) * C::Y_BYTES, yo = yq + C::Y_BYTES;
#pragma unroll
        for (int kk = 0; kk < QT / 16; ++kk)
          umma_bf16(tdV, make_desc(sPm + kk * 2048, 8192, 1024), make_desc(yo + kk * 2048, 8192, 1024), idG,
                    (u | kk) != 0);
#pragma unroll
        for (int kk = 0; kk < QT / 16; ++kk)
          umma_bf16(tdK, make_desc(sdS + kk * 2048, 8192, 1024), make_desc(yq + kk * 2048, 8192, 1024), idG,
                    (u | kk) != 0);
        umma_commit(dsfree);
        umma_commit(yempty(s));
      };
      bool alive = mbar_wait(afull, 0, serr);
      for (int t = 0; t < n_tiles && alive; ++t) {
        const int s = t & 1;
        if (!mbar_wait(yfull(s), (t >> 1) & 1, serr)) { alive = false; break; }
        if (t > 0 && !mbar_wait(sdfree, (t - 1) & 1, serr)) { alive = false; break; }
        tc_fence_after();
        issue_scores(s);
        if (t > 0) {
          if (!mbar_wait(dsfull, (t - 1) & 1, serr)) { alive = false; break; }
          tc_fence_after();
          issue_grads(t - 1);
        }
      }
      if (alive && mbar_wait(dsfull, (n_tiles - 1) & 1, serr)) {
        tc_fence_after();
        issue_grads(n_tiles - 1);
        umma_commit(accdone);
      }
    }
  } else {
    // ---------------- gradient math: one reader row per thread ----------------
    const int q = warp & 3, row = q * 32 + lane;
    const uint32_t tlane = tmem_base + ((uint32_t)(q * 32) << 16);
    auto wwait = [&](uint32_t bar, uint32_t parity) { return __all_sync(0xffffffffu, mbar_wait(bar, parity, serr)); };
    bool alive = n_tiles > 0;
    for (int t = 0; t < n_tiles && alive; ++t) {
      const int qp = s_begin + t * QT + row;               // this thread's reader position
      const bool valid = qp < s_end;
      float L2 = 0.f, cc = 0.f;
      if (valid) {
        const long long idx = ((long long)b * g.T + qp) * g.H + h;
        L2 = lse[idx] * 1.4426950408889634f;
        cc = corr[idx];
      }
      if (!wwait(sdfull, t & 1)) { alive = false; break; }
      tc_fence_after();
      uint32_t pp[32], pds[32];                            // the row's P and dS as bf16 pairs (keys 2i, 2i+1)
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        uint32_t rs[32], rd[32];
        tmem_ld32(tlane + hf * 32, rs);
        tmem_ld32(tlane + 64 + hf * 32, rd);
        tmem_ld_wait();
        if (hf == 1) {
          // S and dP are in registers: the next tile's score products may overwrite them
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(sdfree);
        }
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
          float p[2], w[2];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            float pe = valid ? exp2f(fmaf(__uint_as_float(rs[j + e]), g.scale_log2, -L2)) : 0.f;
            if (g.window && own_pos + hf * 32 + j + e <= qp - g.window) pe = 0.f;
            p[e] = pe;
            w[e] = pe * (__uint_as_float(rd[j + e]) - cc) * g.scale;
          }
          pp[hf * 16 + (j >> 1)] = pack_bf16(p[0], p[1]);
          pds[hf * 16 + (j >> 1)] = pack_bf16(w[0], w[1]);
        }
      }
      // the gradient products of the previous tile must have read dS and P before they are overwritten
      if (t > 0 && !wwait(dsfree, (t - 1) & 1)) { alive = false; break; }
      uint8_t* ds_row = base_ptr + C::ds_off + row * 128;
#pragma unroll
      for (int c8 = 0; c8 < 8; ++c8) {                      // 16-byte chunk c8 = keys [8 c8, 8 c8 + 8), swizzled
        const int off = (c8 ^ (row & 7)) << 4;
        *reinterpret_cast<uint4*>(ds_row + off) = make_uint4(pds[4 * c8], pds[4 * c8 + 1], pds[4 * c8 + 2], pds[4 * c8 + 3]);
        *reinterpret_cast<uint4*>(ds_row + QT * 128 + off) = make_uint4(pp[4 * c8], pp[4 * c8 + 1], pp[4 * c8 + 2], pp[4 * c8 + 3]);
      }
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(dsfull);
    }
    // ---- the accumulated gradients (M = 64 accumulators: rows in lanes 0..15 of each quarter) ----
    const int t4 = lane & 3, rA = q * 16 + (lane >> 2);
    if (alive && n_tiles > 0) alive = wwait(accdone, 0);
    if (alive || n_tiles == 0) {
      if (n_tiles > 0) tc_fence_after();
#pragma unroll 1
      for (int a = 0; a < 2; ++a) {
        float* dstA = (a == 0 ? out1 : out2) + b * g.o_bs + (long long)(z * BT + rA) * g.o_rs + (long long)h * DH;
        float* dstB = dstA + 8 * g.o_rs;
        uint32_t r[32];
        if (n_tiles > 0) {
          tmem_ld_16x256b_x8(tlane + 128 + a * DH, r);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e) r[e] = 0u;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int d = 8 * j + 2 * t4;
          float2 vA = make_float2(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]));
          float2 vB = make_float2(__uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
          if (g.accumulate) {
            const float2 oA = *reinterpret_cast<const float2*>(dstA + d), oB = *reinterpret_cast<const float2*>(dstB + d);
            vA.x += oA.x; vA.y += oA.y; vB.x += oB.x; vB.y += oB.y;
          }
          *reinterpret_cast<float2*>(dstA + d) = vA;
          *reinterpret_cast<float2*>(dstB + d) = vB;
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 256);
  }
  if (threadIdx.x == 0 && *serr) atomicExch(gerr, 1);
}

// ---------------------------------------------------------------------------------------------------------
// Query side with 128 keys per tile (head dim 64): the mirror image of the kernel above.  The group's 64 query
// rows (q, d o) stay in shared memory with their lse / corr (staged once: they do not change from tile to tile);
// the tape's K / V rows stream in tiles of 128.  Scores are formed with the KEYS as the M dimension,
//   S^T = K_t Q^T, dP^T = V_t dO^T    (M = 128, N = 64), one key row per thread,
// dS^T goes to shared memory one 128-byte line per key, and  dQ += dS K_t  reads it as an M-major A operand
// (M = 64 queries, K = 128 keys) against the K tile as an N-major B operand.  Tensor memory: 192 of 256 columns.
struct QCfg {
  static constexpr int O_BYTES = BT * 64 * 2;           // the group's q (or d o): 8 KB
  static constexpr int Y_BYTES = QT * 64 * 2;           // one streamed tile of K (or V): 16 KB
  static constexpr int a_off = 0;
  static constexpr int y_off = 2 * O_BYTES;             // (K, V) x two stages
  static constexpr int ds_off = y_off + 4 * Y_BYTES;    // dS^T [128 keys][64 queries]
  static constexpr int sc_off = ds_off + QT * 128;      // lse (log2 domain) and corr of the 64 queries
  static constexpr int bar_off = sc_off + 512;
  static constexpr int total = bar_off + 256;
};

__global__ void __launch_bounds__(NTHREADS, 2) attn_dq128_tc_kernel(
    const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmDO,
    const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
    const float* __restrict__ lse, const float* __restrict__ corr, float* __restrict__ out1, const BGeo g,
    int* __restrict__ gerr) {
  using C = QCfg;
  constexpr int DH = 64;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t base = smem_u32(smem_raw);
  if (base & 1023u) {
    if (threadIdx.x == 0) atomicExch(gerr, 2);
    return;
  }
  uint8_t* base_ptr = smem_raw;
  const uint32_t bar0 = base + C::bar_off;
  const uint32_t afull = bar0;
  auto yfull = [&](int s) { return bar0 + 8u * (1 + s); };
  auto yempty = [&](int s) { return bar0 + 8u * (3 + s); };
  const uint32_t sdfull = bar0 + 8u * 5, sdfree = bar0 + 8u * 6, dsfull = bar0 + 8u * 7, dsfree = bar0 + 8u * 8,
                 accdone = bar0 + 8u * 9;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(base_ptr + C::bar_off + 8 * 10);
  volatile int* serr = reinterpret_cast<volatile int*>(base_ptr + C::bar_off + 8 * 11);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.x, b = blockIdx.y, z = blockIdx.z, G = gridDim.z;
  const int own_row0 = z * g.grow, own_pos = g.qbase + z * g.grow;
  int s_begin = max(0, g.lo + z * g.grow);
  const int s_end = g.hi + z * g.grow;
  if (g.window) s_begin = min(s_end, max(s_begin, own_pos - g.window + 1));
  const int n_tiles = s_end > s_begin ? (s_end - s_begin + QT - 1) / QT : 0;

  if (threadIdx.x == 0) {
    *serr = 0;
    mbar_init(afull, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(yfull(s), 1);
      mbar_init(yempty(s), 1);
    }
    mbar_init(sdfull, 1);
    mbar_init(sdfree, 4);
    mbar_init(dsfull, 4);
    mbar_init(dsfree, 1);
    mbar_init(accdone, 1);
    fence_barrier_init();
  }
  if (warp == 1) tmem_alloc(tmem_slot, 256);
  // the 64 queries' lse (log2 domain) and corr: dense [B, G, 64, H]
  float* sc = reinterpret_cast<float*>(base_ptr + C::sc_off);
  if (threadIdx.x >= 64 && threadIdx.x < 128) {
    const int r = threadIdx.x - 64;
    const long long idx = ((long long)((b * G + z) * g.C + r) * g.H + h);
    sc[r] = lse[idx] * 1.4426950408889634f;
    sc[64 + r] = corr[idx];
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t sQ = base + C::a_off, sdO = sQ + C::O_BYTES, sY = base + C::y_off, sdS = base + C::ds_off;
  const uint32_t tS = tmem_base, tdP = tmem_base + 64, tdQ = tmem_base + 128;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0 && n_tiles > 0) {
      mbar_expect_tx(afull, 2 * C::O_BYTES);
      tma_load_3d(sQ, &tmQ, afull, h * DH, own_row0, b);
      tma_load_3d(sdO, &tmDO, afull, h * DH, own_row0, b);
      int t = 0;
      for (; t < n_tiles; ++t) {
        const int s = t & 1, r0 = s_begin + t * QT;
        if (!mbar_wait(yempty(s), ((t >> 1) & 1) ^ 1, serr)) break;
        mbar_expect_tx(yfull(s), 2 * C::Y_BYTES);
        tma_load_3d(sY + (2 * s) * C::Y_BYTES, &tmK, yfull(s), h * DH, r0, b);
        tma_load_3d(sY + (2 * s + 1) * C::Y_BYTES, &tmV, yfull(s), h * DH, r0, b);
      }
      if (*serr) {
        volatile int ignore = 0;
        for (int u = max(0, t - 2); u < t; ++u) mbar_wait(yfull(u & 1), (u >> 1) & 1, &ignore);
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0 && n_tiles > 0) {
      constexpr uint32_t idS = instr_desc(QT, BT, 0, 0), idG = instr_desc(BT, DH, 1, 1);
      auto issue_scores = [&](int s) {                      // S^T = K_t Q^T, dP^T = V_t dO^T
        const uint32_t yk = sY + (2 * s) * C::Y_BYTES, yv = yk + C::Y_BYTES;
#pragma unroll
        for (int k = 0; k < DH / 16; ++k)
          umma_bf16(tS, make_desc(yk + k * 32, 16, 1024), make_desc(sQ + k * 32, 16, 1024), idS, k != 0);
#pragma unroll
        for (int k = 0; k < DH / 16; ++k)
          umma_bf16(tdP, make_desc(yv + k * 32, 16, 1024), make_desc(sdO + k * 32, 16, 1024), idS, k != 0);
        umma_commit(sdfull);
      };
      auto issue_grads = [&](int u) {                       // dQ += dS K_t of tile u
        const int s = u & 1;
        const uint32_t yk = sY + (2 * s) * C::Y_BYTES;
#pragma unroll
        for (int kk = 0; kk < QT / 16; ++kk)
          umma_bf16(tdQ, make_desc(sdS + kk * 2048, 8192, 1024), make_desc(yk + kk * 2048, 8192, 1024), idG,
                    (u | kk) != 0);
        umma_commit(dsfree);
        umma_commit(yempty(s));
      };
      bool alive = mbar_wait(afull, 0, serr);
      for (int t = 0; t < n_tiles && alive; ++t) {
        const int s = t & 1;
        if (!mbar_wait(yfull(s), (t >> 1) & 1, serr)) { alive = false; break; }
        if (t > 0 && !mbar_wait(sdfree, (t - 1) & 1, serr)) { alive = false; break; }
        tc_fence_after();
        issue_scores(s);
        if (t > 0) {
          if (!mbar_wait(dsfull, (t - 1) & 1, serr)) { alive = false; break; }
          tc_fence_after();
          issue_grads(t - 1);
        }
      }
      if (alive && mbar_wait(dsfull, (n_tiles - 1) & 1, serr)) {
        tc_fence_after();
        issue_grads(n_tiles - 1);
        umma_commit(accdone);
      }
    }
  } else {
    // ---------------- gradient math: one key row per thread ----------------
    const int q = warp & 3, row = q * 32 + lane;
    const uint32_t tlane = tmem_base + ((uint32_t)(q * 32) << 16);
    auto wwait = [&](uint32_t bar, uint32_t parity) { return __all_sync(0xffffffffu, mbar_wait(bar, parity, serr)); };
    bool alive = n_tiles > 0;
    for (int t = 0; t < n_tiles && alive; ++t) {
      const int kp = s_begin + t * QT + row;               // this thread's key (tape row)
      const bool valid = kp < s_end;
      if (!wwait(sdfull, t & 1)) { alive = false; break; }
      tc_fence_after();
      uint32_t pds[32];                                    // the key's dS over the 64 queries as bf16 pairs
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        uint32_t rs[32], rd[32];
        tmem_ld32(tlane + hf * 32, rs);
        tmem_ld32(tlane + 64 + hf * 32, rd);
        tmem_ld_wait();
        if (hf == 1) {
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(sdfree);
        }
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
          const int c = hf * 32 + j;
          const float2 L2 = *reinterpret_cast<const float2*>(sc + c), cc = *reinterpret_cast<const float2*>(sc + 64 + c);
          float w[2];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            float pe = valid ? exp2f(fmaf(__uint_as_float(rs[j + e]), g.scale_log2, -(e ? L2.y : L2.x))) : 0.f;
            if (g.window && kp <= own_pos + c + e - g.window) pe = 0.f;
            w[e] = pe * (__uint_as_float(rd[j + e]) - (e ? cc.y : cc.x)) * g.scale;
          }
          pds[hf * 16 + (j >> 1)] = pack_bf16(w[0], w[1]);
        }
      }
      if (t > 0 && !wwait(dsfree, (t - 1) & 1)) { alive = false; break; }
      uint8_t* ds_row = base_ptr + C::ds_off + row * 128;
#pragma unroll
      for (int c8 = 0; c8 < 8; ++c8)
        *reinterpret_cast<uint4*>(ds_row + ((c8 ^ (row & 7)) << 4)) =
            make_uint4(pds[4 * c8], pds[4 * c8 + 1], pds[4 * c8 + 2], pds[4 * c8 + 3]);
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(dsfull);
    }
    // ---- d q (M = 64 accumulator: rows in lanes 0..15 of each quarter) ----
    const int t4 = lane & 3, rA = q * 16 + (lane >> 2);
    if (alive && n_tiles > 0) alive = wwait(accdone, 0);
    if (alive || n_tiles == 0) {
      if (n_tiles > 0) tc_fence_after();
      float* dstA = out1 + b * g.o_bs + (long long)(z * BT + rA) * g.o_rs + (long long)h * DH;
      float* dstB = dstA + 8 * g.o_rs;
      uint32_t r[32];
      if (n_tiles > 0) {
        tmem_ld_16x256b_x8(tlane + 128, r);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int e = 0; e < 32; ++e) r[e] = 0u;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int d = 8 * j + 2 * t4;
        float2 vA = make_float2(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]));
        float2 vB = make_float2(__uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
        if (g.accumulate) {
          const float2 oA = *reinterpret_cast<const float2*>(dstA + d), oB = *reinterpret_cast<const float2*>(dstB + d);
          vA.x += oA.x; vA.y += oA.y; vB.x += oB.x; vB.y += oB.y;
        }
        *reinterpret_cast<float2*>(dstA + d) = vA;
        *reinterpret_cast<float2*>(dstB + d) = vB;
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 256);
  }
  if (threadIdx.x == 0 && *serr) atomicExch(gerr, 1);
}

template <int DH, int KEYSIDE>
int launch_bwd(const CUtensorMap& a1, const CUtensorMap& a2, const CUtensorMap& y1, const CUtensorMap& y2,
               const float* lse, const float* corr, float* out1, float* out2, int B, int G, const BGeo& g, int* gerr,
               cudaStream_t st) {
  using C = BCfg<DH, KEYSIDE>;
  auto kern = attn_bwd_tc_kernel<DH, KEYSIDE>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::total);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  kern<<<dim3(g.H, B, G), NTHREADS, C::total, st>>>(a1, a2, y1, y2, lse, corr, out1, out2, g, gerr);
  DMB_CHECK_LAUNCH();
  return 0;
}

int g_dkv_rows128 = 1;

}  // namespace

extern "C" {

// Query side of the read's backward.  q, do_c: bf16 views [B, rows, H, DH] (group z: rows [z*grow, z*grow + 64));
// keys of group z: tape rows max(0, lo + z*grow) <= j < hi + z*grow; query row i sits at qbase + z*grow + i;
// lse, corr: dense [B, G, 64, H] fp32; dq: fp32 view [B, G*64, H, DH] with strides vdq, added to when accumulate != 0.
int dmb_attn_dq_tc(const void* q, TView vq, const void* do_c, TView vdo, int q_rows, const void* Kc, const void* Vc,
                   TView vc, int tape_rows, const float* lse, const float* corr, float* dq, TView vdq, int B, int G, int H,
                   int dh, int lo, int hi, int qbase, int grow, float scale, int window, int accumulate, int* gerr,
                   cudaStream_t st) {
  if (!encode_fn()) return -10;
  if ((dh != 64 && dh != 128) || B <= 0 || G <= 0) return -1;
  BGeo g = {};
  g.H = H; g.C = BT; g.lo = lo; g.hi = hi; g.qbase = qbase; g.grow = grow; g.window = window; g.accumulate = accumulate;
  g.o_bs = vdq.bs; g.o_rs = vdq.rs;
  g.scale = scale; g.scale_log2 = scale * 1.4426950408889634f;
  const long long cols = (long long)H * dh;
  const int k_rows = max(1, min(tape_rows, hi + (G - 1) * grow));
  CUtensorMap a1, a2, y1, y2;
  int rc;
  if ((rc = make_map_3d(&a1, q, cols, q_rows, B, vq.rs, B > 1 ? vq.bs : (long long)q_rows * vq.rs, 64, 64))) return rc;
  if ((rc = make_map_3d(&a2, do_c, cols, q_rows, B, vdo.rs, B > 1 ? vdo.bs : (long long)q_rows * vdo.rs, 64, 64))) return rc;
  const long long kbs = B > 1 ? vc.bs : (long long)tape_rows * vc.rs;
  if ((rc = make_map_3d(&y1, Kc, cols, k_rows, B, vc.rs, kbs, 64, 64))) return rc;
  if ((rc = make_map_3d(&y2, Vc, cols, k_rows, B, vc.rs, kbs, 64, 64))) return rc;
  if (dh == 64 && g_dkv_rows128) {
    // 128 keys per streamed tile: the same tape maps with a taller box
    if ((rc = make_map_3d(&y1, Kc, cols, k_rows, B, vc.rs, kbs, 64, QT))) return rc;
    if ((rc = make_map_3d(&y2, Vc, cols, k_rows, B, vc.rs, kbs, 64, QT))) return rc;
    static bool configured = false;
    if (!configured) {
      cudaError_t e = cudaFuncSetAttribute(attn_dq128_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, QCfg::total);
      if (e != cudaSuccess) return (int)e;
      configured = true;
    }
    attn_dq128_tc_kernel<<<dim3(H, B, G), NTHREADS, QCfg::total, st>>>(a1, a2, y1, y2, lse, corr, dq, g, gerr);
    DMB_CHECK_LAUNCH();
    return 0;
  }
  if (dh == 64) return launch_bwd<64, 0>(a1, a2, y1, y2, lse, corr, dq, nullptr, B, G, g, gerr, st);
  return launch_bwd<128, 0>(a1, a2, y1, y2, lse, corr, dq, nullptr, B, G, g, gerr, st);
}

// Key side.  Chunk z owns the tape rows [pos0 + z*grow, + 64) of Kc / Vc; its readers are the query positions
// [max(q_start, chunk end), min(q_end, chunk start + span)) of q_all / doc_all (dense [B, T, H, DH] bf16) with
// lse_all / corr_all dense [B, T, H] fp32.  dK, dV: fp32 views [B, G*64, H, DH] with strides vdkv (chunk z at rows
// z*64), written, or added to when accumulate != 0.
int dmb_attn_dkv_tc(const void* q_all, const void* doc_all, const float* corr_all, const float* lse_all, int T,
                    const void* Kc, const void* Vc, TView vc, int tape_rows, float* dK, float* dV, TView vdkv, int accumulate,
                    int B, int G, int H, int dh, int pos0, int q_start, int q_end, int grow, int span, float scale,
                    int window, int* gerr, cudaStream_t st) {
  if (!encode_fn()) return -10;
  if ((dh != 64 && dh != 128) || B <= 0 || G <= 0) return -1;
  BGeo g = {};
  g.H = H; g.T = T; g.C = BT; g.lo = pos0; g.grow = grow; g.window = window; g.span = span;
  g.q_start = q_start; g.q_end = min(q_end, T); g.accumulate = accumulate; g.o_bs = vdkv.bs; g.o_rs = vdkv.rs; g.scale = scale; g.scale_log2 = scale * 1.4426950408889634f;
  const long long cols = (long long)H * dh;
  CUtensorMap a1, a2, y1, y2;
  int rc;
  const long long kbs = B > 1 ? vc.bs : (long long)tape_rows * vc.rs;
  if ((rc = make_map_3d(&a1, Kc, cols, tape_rows, B, vc.rs, kbs, 64, 64))) return rc;
  if ((rc = make_map_3d(&a2, Vc, cols, tape_rows, B, vc.rs, kbs, 64, 64))) return rc;
  // query rows at and beyond q_end are outside the maps: zero-filled
  const int y_rows = max(1, g.q_end);
  if ((rc = make_map_3d(&y1, q_all, cols, y_rows, B, cols, (long long)T * cols, 64, 64))) return rc;
  if ((rc = make_map_3d(&y2, doc_all, cols, y_rows, B, cols, (long long)T * cols, 64, 64))) return rc;
  if (dh == 64 && g_dkv_rows128) {
    // 128 reader rows per streamed tile: the same maps with a taller box
    if ((rc = make_map_3d(&y1, q_all, cols, y_rows, B, cols, (long long)T * cols, 64, QT))) return rc;
    if ((rc = make_map_3d(&y2, doc_all, cols, y_rows, B, cols, (long long)T * cols, 64, QT))) return rc;
    static bool configured = false;
    if (!configured) {
      cudaError_t e = cudaFuncSetAttribute(attn_dkv128_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, KCfg::total);
      if (e != cudaSuccess) return (int)e;
      configured = true;
    }
    attn_dkv128_tc_kernel<<<dim3(H, B, G), NTHREADS, KCfg::total, st>>>(a1, a2, y1, y2, lse_all, corr_all, dK, dV, g, gerr);
    DMB_CHECK_LAUNCH();
    return 0;
  }
  if (dh == 64) return launch_bwd<64, 1>(a1, a2, y1, y2, lse_all, corr_all, dK, dV, B, G, g, gerr, st);
  return launch_bwd<128, 1>(a1, a2, y1, y2, lse_all, corr_all, dK, dV, B, G, g, gerr, st);
}

// 1 (default): at head dim 64 the key side streams its readers, and the query side its keys, in tiles of 128 rows;
// 0: in tiles of 64
int dmb_attn_dkv_rows128(int on) {
  const int was = g_dkv_rows128;
  if (on >= 0) g_dkv_rows128 = on;
  return was;
}

}  // extern "C"
