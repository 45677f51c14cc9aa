// Flash-style attention forward on the 5th-generation tensor cores.
//
// One CTA per (batch, head, tile of BM query rows).  Keys and values stream from a token-major tape
// [B, T, H, DH] in tiles of 128 rows:
//
//   warp 0      TMA producer: Q once, then K / V tiles into a two-stage ring (128-byte swizzle)
//   warp 1      one thread issues  S = Q K^T  (tcgen05.mma, M = BM, N = 128, fp32 in TMEM) and
//               O_t = P V  (M = BM, N = DH) per key tile; the accumulators live in tensor memory
//   warps 2..5  softmax: every thread owns one query row (its TMEM lane).  It reads S with
//               tcgen05.ld, masks, keeps the running maximum and sum in the log2 domain, writes
//               P = exp2(S - m) as bf16 into shared memory in the operand layout of the second
//               product, and folds the product of the previous tile (read back from TMEM, two buffers)
//               into its fp32 output row with the usual rescale.
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
  int H, Lq, lo, hi, qbase, grow, window, causal, causal_excl, tiles_q, lane_mode, o_bf16;
  float scale_log2;
};

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
  int k_begin = lo_z, k_end = hi_z;
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
    // row of the tile held by this thread's TMEM lane.  M = 128: lane l of the accumulator is row l.
    // M = 64: lane_mode 0: rows 16q..16q+15 sit in lanes 32q..32q+15; lane_mode 1: row r sits in lane r.
    int row;
    bool has_row;
    if (BM == 128) {
      row = q * 32 + lane;
      has_row = true;
    } else if (g.lane_mode == 0) {
      row = q * 16 + lane;
      has_row = lane < 16;
    } else {
      row = q * 32 + lane;
      has_row = q < 2;
    }
    const uint32_t tlane = tmem_base + ((uint32_t)(q * 32) << 16);
    const int qpos = qpos0 + row;
    int jlo = lo_z, jhi = hi_z;                              // allowed keys of this row: jlo <= j < jhi
    if (g.window) jlo = max(jlo, qpos - g.window + 1);
    if (g.causal) jhi = min(jhi, qpos - g.causal_excl + 1);
    float m = -INFINITY, l = 0.f, alpha_prev = 1.f;
    float O[DH];
#pragma unroll
    for (int d = 0; d < DH; ++d) O[d] = 0.f;
    uint8_t* pP = base_ptr + C::p_off;
    bool alive = n_tiles > 0;
    auto fold = [&](int u, float alpha) {                    // O = O * alpha + (P V) of tile u
      const int s = u & 1;
      if (!mbar_wait(pvfull(s), (u >> 1) & 1, serr)) return false;
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
      if (!mbar_wait(sfull, t & 1, serr)) { alive = false; break; }
      tc_fence_after();
      // a tile needs per-element masks only where it crosses a row's range
      const bool mask = (k0 + KT > k_end) || (k0 < lo_z) || (g.causal && k0 + KT - 1 > qpos0 - g.causal_excl) ||
                        (g.window && k0 < qpos0 + rows_here - 1 - g.window + 1);
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
      if (g.o_bf16) {
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
      lse_out[orow] = l > 0.f ? (m + log2f(l)) * 0.6931471805599453f : DMB_NEG;
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
  const int k_rows = max(1, min(tape_rows, g.hi + (G - 1) * g.grow));
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
//   bm: 64 or 128 query rows per CTA.  lane_mode: how the M = 64 accumulator maps to TMEM lanes (0: 16 rows
//   per 32-lane quarter).  gerr: device int, set to 1 if a pipeline wait ran out.
// Requirements: 16-byte aligned pointers, strides multiples of 8 elements, dh 64 or 128.
int dmb_attn_fwd_tc(const void* q, TView vq, int q_rows, const void* Kc, const void* Vc, TView vc, int tape_rows,
                    void* o, int o_bf16, float* lse, int B, int G, int Lq, int H, int dh, int lo, int hi, int qbase,
                    int grow, float scale, int window, int causal, int causal_excl, int bm, int lane_mode, int* gerr,
                    cudaStream_t st) {
  if (!encode_fn()) return -10;
  if ((dh != 64 && dh != 128) || (bm != 64 && bm != 128) || Lq <= 0 || B <= 0 || G <= 0) return -1;
  Geo g;
  g.H = H; g.Lq = Lq; g.lo = lo; g.hi = hi; g.qbase = qbase; g.grow = grow; g.window = window;
  g.causal = causal; g.causal_excl = causal_excl; g.tiles_q = (Lq + bm - 1) / bm; g.lane_mode = lane_mode;
  g.o_bf16 = o_bf16; g.scale_log2 = scale * 1.4426950408889634f;
  if (dh == 64) {
    if (bm == 64) return launch<64, 64>(q, vq, q_rows, Kc, Vc, vc, tape_rows, o, lse, B, G, g, gerr, st);
    return launch<64, 128>(q, vq, q_rows, Kc, Vc, vc, tape_rows, o, lse, B, G, g, gerr, st);
  }
  if (bm == 64) return launch<128, 64>(q, vq, q_rows, Kc, Vc, vc, tape_rows, o, lse, B, G, g, gerr, st);
  return launch<128, 128>(q, vq, q_rows, Kc, Vc, vc, tape_rows, o, lse, B, G, g, gerr, st);
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
// 0..15 of each 32-lane quarter, so lanes 16..31 of the four math warps only take part in the collective
// tensor-memory loads.  Tensor memory: S 64 | dP 64 | accumulators: 256 columns at head dim 64 (two CTAs
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
    // ---------------- gradient math: one owner row per thread ----------------
    const int q = warp & 3;
    const int row = q * 16 + lane;
    const bool has_row = lane < 16;
    const uint32_t tlane = tmem_base + ((uint32_t)(q * 32) << 16);
    const int rpos = own_pos + row;                          // absolute position of this owner row
    // dense per-row arrays of the query side: [B, G, C, H]
    const long long orow = ((long long)((b * G + z) * g.C + row) * g.H + h);
    float L2r = 0.f, cr = 0.f;
    if (!KEYSIDE && has_row) {
      L2r = lse[orow] * 1.4426950408889634f;
      cr = corr[orow];
    }
    // every math warp stages its own copy of the per-column scalars, so no barrier spans the warps
    float* sc = reinterpret_cast<float*>(base_ptr + C::sc_off) + q * 256;
    uint8_t* pdS = base_ptr + C::ds_off;
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
      if (!mbar_wait(sdfull, t & 1, serr)) { alive = false; break; }
      tc_fence_after();
      uint32_t rs[64], rd[64];
      tmem_ld32(tlane, *reinterpret_cast<uint32_t (*)[32]>(&rs[0]));
      tmem_ld32(tlane + 32, *reinterpret_cast<uint32_t (*)[32]>(&rs[32]));
      tmem_ld32(tlane + 64, *reinterpret_cast<uint32_t (*)[32]>(&rd[0]));
      tmem_ld32(tlane + 96, *reinterpret_cast<uint32_t (*)[32]>(&rd[32]));
      tmem_ld_wait();
      // S and dP are in registers: the next tile's score products may overwrite them
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(sdfree);
      const bool mask = (c0pos + BT > s_end) || g.window != 0;
      uint32_t pds[32], pp[32];
      const float* scL = sc + (t & 1) * 128;
#pragma unroll
      for (int e = 0; e < 64; e += 2) {
        float v[2], w[2];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const float L2 = KEYSIDE ? scL[e + u] : L2r, cc = KEYSIDE ? scL[64 + e + u] : cr;
          float p = exp2f(fmaf(__uint_as_float(rs[e + u]), g.scale_log2, -L2));
          if (mask) {
            const int cpos = c0pos + e + u;
            const int key = KEYSIDE ? rpos : cpos, qp = KEYSIDE ? cpos : rpos;
            if (cpos >= s_end || (g.window && key <= qp - g.window)) p = 0.f;
          }
          v[u] = p;
          w[u] = p * (__uint_as_float(rd[e + u]) - cc) * g.scale;
        }
        pds[e >> 1] = pack_bf16(w[0], w[1]);
        if (KEYSIDE) pp[e >> 1] = pack_bf16(v[0], v[1]);
      }
      // the gradient products of the previous tile must have read dS (and P) before they are overwritten
      if (t > 0 && !mbar_wait(dsfree, (t - 1) & 1, serr)) { alive = false; break; }
      if (has_row) {
        uint8_t* rowp = pdS + row * 128;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          *reinterpret_cast<uint4*>(rowp + ((c ^ (row & 7)) << 4)) =
              make_uint4(pds[4 * c], pds[4 * c + 1], pds[4 * c + 2], pds[4 * c + 3]);
          if (KEYSIDE)
            *reinterpret_cast<uint4*>(rowp + BT * 128 + ((c ^ (row & 7)) << 4)) =
                make_uint4(pp[4 * c], pp[4 * c + 1], pp[4 * c + 2], pp[4 * c + 3]);
        }
      }
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(dsfull);
    }
    // ---- the accumulated gradients ----
    if (alive && n_tiles > 0) alive = mbar_wait(accdone, 0, serr);
    if (alive || n_tiles == 0) {
      if (n_tiles > 0) tc_fence_after();
      const long long drow = orow * DH;                      // dense [B, G, C, H, DH] for both sides
#pragma unroll 1
      for (int a = 0; a < (KEYSIDE ? 2 : 1); ++a) {
        float* dst = (a == 0 ? out1 : out2) + drow;
#pragma unroll 1
        for (int c0 = 0; c0 < DH; c0 += 64) {
          uint32_t r[64];
          if (n_tiles > 0) {
            tmem_ld32(tlane + 128 + a * DH + c0, *reinterpret_cast<uint32_t (*)[32]>(&r[0]));
            tmem_ld32(tlane + 128 + a * DH + c0 + 32, *reinterpret_cast<uint32_t (*)[32]>(&r[32]));
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int e = 0; e < 64; ++e) r[e] = 0u;
          }
          if (has_row) {
#pragma unroll
            for (int e = 0; e < 64; e += 4) {
              float4 v = make_float4(__uint_as_float(r[e]), __uint_as_float(r[e + 1]), __uint_as_float(r[e + 2]),
                                     __uint_as_float(r[e + 3]));
              if (g.accumulate) {
                const float4 o = *reinterpret_cast<const float4*>(dst + c0 + e);
                v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
              }
              *reinterpret_cast<float4*>(dst + c0 + e) = v;
            }
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

}  // namespace

extern "C" {

// Query side of the read's backward.  q, do_c: bf16 views [B, rows, H, DH] (group z: rows [z*grow, z*grow + 64));
// keys of group z: tape rows max(0, lo + z*grow) <= j < hi + z*grow; query row i sits at qbase + z*grow + i;
// lse, corr: dense [B, G, 64, H] fp32; dq: dense [B, G, 64, H, DH] fp32, added to when accumulate != 0.
int dmb_attn_dq_tc(const void* q, TView vq, const void* do_c, TView vdo, int q_rows, const void* Kc, const void* Vc,
                   TView vc, int tape_rows, const float* lse, const float* corr, float* dq, int B, int G, int H, int dh,
                   int lo, int hi, int qbase, int grow, float scale, int window, int accumulate, int* gerr,
                   cudaStream_t st) {
  if (!encode_fn()) return -10;
  if ((dh != 64 && dh != 128) || B <= 0 || G <= 0) return -1;
  BGeo g = {};
  g.H = H; g.C = BT; g.lo = lo; g.hi = hi; g.qbase = qbase; g.grow = grow; g.window = window; g.accumulate = accumulate;
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
  if (dh == 64) return launch_bwd<64, 0>(a1, a2, y1, y2, lse, corr, dq, nullptr, B, G, g, gerr, st);
  return launch_bwd<128, 0>(a1, a2, y1, y2, lse, corr, dq, nullptr, B, G, g, gerr, st);
}

// Key side.  Chunk z owns the tape rows [pos0 + z*grow, + 64) of Kc / Vc; its readers are the query positions
// [max(q_start, chunk end), min(q_end, chunk start + span)) of q_all / doc_all (dense [B, T, H, DH] bf16) with
// lse_all / corr_all dense [B, T, H] fp32.  dK, dV: dense [B, G, 64, H, DH] fp32, written.
int dmb_attn_dkv_tc(const void* q_all, const void* doc_all, const float* corr_all, const float* lse_all, int T,
                    const void* Kc, const void* Vc, TView vc, int tape_rows, float* dK, float* dV, int B, int G, int H,
                    int dh, int pos0, int q_start, int q_end, int grow, int span, float scale, int window, int* gerr,
                    cudaStream_t st) {
  if (!encode_fn()) return -10;
  if ((dh != 64 && dh != 128) || B <= 0 || G <= 0) return -1;
  BGeo g = {};
  g.H = H; g.T = T; g.C = BT; g.lo = pos0; g.grow = grow; g.window = window; g.span = span;
  g.q_start = q_start; g.q_end = min(q_end, T); g.scale = scale; g.scale_log2 = scale * 1.4426950408889634f;
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
  if (dh == 64) return launch_bwd<64, 1>(a1, a2, y1, y2, lse_all, corr_all, dK, dV, B, G, g, gerr, st);
  return launch_bwd<128, 1>(a1, a2, y1, y2, lse_all, corr_all, dK, dV, B, G, g, gerr, st);
}

}  // extern "C"
