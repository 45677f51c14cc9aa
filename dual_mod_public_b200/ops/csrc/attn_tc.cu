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
__global__ void __launch_bounds__(NTHREADS) attn_fwd_tc_kernel(
    const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
    const __grid_constant__ CUtensorMap tmV, void* __restrict__ o_out, float* __restrict__ lse_out,
    const Geo g, int* __restrict__ gerr) {
  using C = Cfg<DH, BM>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
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
      for (int c0 = 0; c0 < DH; c0 += 32) {
        uint32_t r[32];
        tmem_ld32(tlane + KT + s * DH + c0, r);
        tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < 32; ++e) O[c0 + e] = O[c0 + e] * alpha + __uint_as_float(r[e]);
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
      for (int c0 = 0; c0 < KT; c0 += 32) {
        uint32_t r[32];
        tmem_ld32(tlane + c0, r);
        tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          const int j = k0 + c0 + e;
          const float v = __uint_as_float(r[e]);
          mx = fmaxf(mx, (!mask || (j >= jlo && j < jhi)) ? v : -INFINITY);
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
      for (int c0 = 0; c0 < KT; c0 += 32) {
        uint32_t r[32];
        tmem_ld32(tlane + c0, r);
        tmem_ld_wait();
        uint32_t pk[16];
#pragma unroll
        for (int e = 0; e < 32; e += 2) {
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
          const int ch0 = (c0 & 63) >> 3;
#pragma unroll
          for (int c = 0; c < 4; ++c)
            *reinterpret_cast<uint4*>(rowp + (((ch0 + c) ^ (row & 7)) << 4)) =
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
  const int smem = C::total + 1024;
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
  const int k_rows = min(tape_rows, g.hi + (G - 1) * g.grow);
  if (k_rows <= 0) return -1;
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
