// bf16 GEMM for problems with few output tiles and a long reduction (the input gradient of a sweep:
// 2048 x 1024 outputs over K = 4096 is 64 tiles of 128 x 256 for 148 SMs): two CTAs of a cluster share one
// 128 x 256 tile and split its K range in halves.  Narrow tiles do not help here (a 128 x 128 x 16 MMA takes as
// long as a 128 x 256 x 16 one), and partial sums through global memory plus a second launch cost more than they save.
//
//   C[M,N] = op(A) . op(B) (+ bias)      bf16 operands and result, fp32 accumulate; layouts as in the single-CTA kernel
//
// Both CTAs run the usual pipeline over their half of the k-blocks (warp 0 = TMA producer, warp 1 = MMA issuer and
// tensor-memory owner, warps 2..9 = epilogue) with the accumulator in their own tensor memory.  Then each CTA's
// epilogue warps write the 128 columns the PARTNER finalises, as fp32, into the partner's shared memory (its operand
// ring, free by then; 16 bytes per lane, lanes on consecutive rows), add the partner's partial to their own 128
// columns and store them through swizzled staging slots and TMA stores.  Hand-shakes per direction: "my ring is
// free" (my MMAs are complete) and, from the eight sending warps, "your partial is written".
// Every wait is bounded in time; on expiry the kernel raises the error flag, stops waiting and runs to its end
// (tensor memory released, the pair leaves together).
#include "tc05.cuh"

using namespace tc05;

namespace {

constexpr int BM = 128, BN = 256, BK = 64, UMMA_K = 16, STAGES = 4;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int NTHREADS = 320, TMEM_COLS = BN;      // producer, MMA issuer, eight epilogue warps
constexpr int stage_out_off = STAGES * STAGE_BYTES;          // epilogue staging: 8 warps x 4 KB
constexpr int bar_off = stage_out_off + 8 * 4096;
constexpr int SMEM_TOTAL = bar_off + 256;
static_assert(BM * (BN / 2) * 4 <= STAGES * STAGE_BYTES, "the partner's partial must fit in the operand ring");

template <int A_MN, int B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NTHREADS, 1) gemm_ksplit2_kernel(
    const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
    const __grid_constant__ CUtensorMap tmC, const bf16* __restrict__ bias, int M, int N, int K,
    int* __restrict__ gerr) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t base = smem_u32(smem_raw);
  uint8_t* base_ptr = smem_raw;
  const uint32_t bar0 = base + bar_off;
  // barriers (same offsets in both CTAs): full[s], empty[s], accumulator complete, partner's ring free, partner's
  // partial written into this CTA's ring; then the TMEM address slot and the error word
  auto full = [&](int s) { return bar0 + 8u * s; };
  auto empty = [&](int s) { return bar0 + 8u * (STAGES + s); };
  const uint32_t tmem_full = bar0 + 8u * (2 * STAGES), ring_free = bar0 + 8u * (2 * STAGES + 1),
                 partial_full = bar0 + 8u * (2 * STAGES + 2);
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(base_ptr + bar_off + 8 * (2 * STAGES + 3));
  volatile int* serr = reinterpret_cast<volatile int*>(base_ptr + bar_off + 8 * (2 * STAGES + 4));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();
  const int tile = blockIdx.x >> 1;
  const int tiles_n = (N + BN - 1) / BN;
  const int m0 = (tile / tiles_n) * BM, n0 = (tile % tiles_n) * BN;
  const int KBT = (K + BK - 1) / BK, KBS = (KBT + 1) / 2;
  const int kb0 = (int)rank * KBS, kb1 = min(KBT, kb0 + KBS);     // the host refuses K < 8 k-blocks: never empty
  const bool aligned = (base & 1023u) == 0;

  if (threadIdx.x == 0) {
    *serr = aligned ? 0 : 1;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full(s), 1);
      mbar_init(empty(s), 1);
    }
    mbar_init(tmem_full, 1);
    mbar_init(ring_free, 1);
    mbar_init(partial_full, 8);          // one arrival per epilogue warp of the partner
    fence_barrier_init();
  }
  if (warp == 1) tmem_alloc(tmem_slot, TMEM_COLS);
  tc_fence_before();
  cluster_sync_all();                    // the partner's barriers exist before anything arrives on them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0 && aligned) {
      uint32_t it = 0;
      for (int kb = kb0; kb < kb1; ++kb, ++it) {
        const int s = it % STAGES;
        if (!mbar_wait(empty(s), ((it / STAGES) & 1) ^ 1, serr)) break;
        const uint32_t sa = base + s * STAGE_BYTES, sb = sa + A_BYTES;
        mbar_expect_tx(full(s), STAGE_BYTES);
        const int k0 = kb * BK;
        if (A_MN == 0) {
          tma_load_2d(sa, &tmA, full(s), k0, m0);                       // box {64 k, 128 m}
        } else {
#pragma unroll
          for (int j = 0; j < BM / 64; ++j) tma_load_2d(sa + j * (BK * 128), &tmA, full(s), m0 + 64 * j, k0);
        }
        if (B_MN == 0) {
          tma_load_2d(sb, &tmB, full(s), k0, n0);                       // box {64 k, 256 n}
        } else {
#pragma unroll
          for (int j = 0; j < BN / 64; ++j) tma_load_2d(sb + j * (BK * 128), &tmB, full(s), n0 + 64 * j, k0);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0 && aligned) {
      constexpr uint32_t idesc = instr_desc(BM, BN, A_MN, B_MN);
      uint32_t it = 0;
      bool alive = true;
      for (int kb = kb0; kb < kb1; ++kb, ++it) {
        const int s = it % STAGES;
        if (!mbar_wait(full(s), (it / STAGES) & 1, serr)) { alive = false; break; }
        tc_fence_after();
        const uint32_t sa = base + s * STAGE_BYTES, sb = sa + A_BYTES;
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k) {
          const uint64_t da = A_MN == 0 ? make_desc(sa + k * 32, 16, 1024) : make_desc(sa + k * 2048, BK * 128, 1024);
          const uint64_t db = B_MN == 0 ? make_desc(sb + k * 32, 16, 1024) : make_desc(sb + k * 2048, BK * 128, 1024);
          umma_bf16(tmem_base, da, db, idesc, ((kb - kb0) | k) != 0);
        }
        umma_commit(empty(s));
      }
      if (alive) umma_commit(tmem_full);       // this CTA's half of the sum is complete, its ring is read
    }
  } else {
    // ---------------- epilogue warps (eight: two per TMEM lane quarter, 64 columns each) ----------------
    // CTA r finalises columns [128 r, 128 r + 128) of the tile: it sends the other 128 columns of its accumulator to
    // the partner and adds the partner's partial to its own columns.
    const int e = warp - 2, q = warp & 3, g = e >> 2;      // q: TMEM lane quarter this warp may touch; g: column half
    const uint32_t peer = rank ^ 1u;
    const int own0 = (int)rank * (BN / 2) + g * 64, send0 = (int)peer * (BN / 2) + g * 64;
    bool alive = aligned && mbar_wait(tmem_full, 0, serr);
    tc_fence_after();
    // this CTA's MMAs are complete, so its operand ring may be overwritten by the partner
    if (e == 0 && lane == 0 && alive) mbar_arrive_cluster(map_to_cta(ring_free, peer));
    alive = alive && mbar_wait_cluster(ring_free, 0, serr);
    if (alive) {
      // rows q*32 + lane, 64 columns, into the partner's ring as [column / 4][row][4] fp32 (16 bytes per lane)
      const uint32_t dst0 = map_to_cta(base, peer) + (uint32_t)(g * 16) * (BM * 16) + (uint32_t)(q * 32 + lane) * 16u;
#pragma unroll
      for (int c0 = 0; c0 < 64; c0 += 32) {
        uint32_t r[32];
        tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + send0 + c0, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; j += 4)
          st_cluster_v4(dst0 + (uint32_t)((c0 + j) >> 2) * (BM * 16), r[j], r[j + 1], r[j + 2], r[j + 3]);
      }
    }
    asm volatile("fence.acq_rel.cluster;" ::: "memory");
    __syncwarp();
    if (lane == 0 && alive) mbar_arrive_cluster(map_to_cta(partial_full, peer));
    alive = alive && mbar_wait_cluster(partial_full, 0, serr);
    const int col = n0 + own0;
    if (alive && m0 + q * 32 < M && col < N) {         // warp-uniform
      const float4* part = reinterpret_cast<const float4*>(base_ptr) + (g * 16) * BM + (q * 32 + lane);
      uint32_t r[64];
      {
        uint32_t (&ra)[32] = *reinterpret_cast<uint32_t (*)[32]>(&r[0]);
        uint32_t (&rb)[32] = *reinterpret_cast<uint32_t (*)[32]>(&r[32]);
        tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + own0, ra);
        tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + own0 + 32, rb);
      }
      tmem_ld_wait();
      uint8_t* slot = base_ptr + stage_out_off + e * 4096;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float4 p0 = part[(2 * j) * BM], p1 = part[(2 * j + 1) * BM];
        float f[8] = {__uint_as_float(r[j * 8]) + p0.x,     __uint_as_float(r[j * 8 + 1]) + p0.y,
                      __uint_as_float(r[j * 8 + 2]) + p0.z, __uint_as_float(r[j * 8 + 3]) + p0.w,
                      __uint_as_float(r[j * 8 + 4]) + p1.x, __uint_as_float(r[j * 8 + 5]) + p1.y,
                      __uint_as_float(r[j * 8 + 6]) + p1.z, __uint_as_float(r[j * 8 + 7]) + p1.w};
        if (bias) {
#pragma unroll
          for (int i = 0; i < 8; ++i)
            if (col + j * 8 + i < N) f[i] += __bfloat162float(bias[col + j * 8 + i]);
        }
        const uint4 o = make_uint4(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]), pack_bf16(f[4], f[5]), pack_bf16(f[6], f[7]));
        // 128-byte swizzle: 16-byte chunk j of row `lane` sits at chunk j ^ (lane & 7)
        *reinterpret_cast<uint4*>(slot + lane * 128 + ((j ^ (lane & 7)) << 4)) = o;
      }
      fence_async_smem();
      __syncwarp();
      if (lane == 0) {
        tma_store_2d(&tmC, smem_u32(slot), col, m0 + q * 32);
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");              // the store completes before exit
      }
    }
  }
  tc_fence_before();
  cluster_sync_all();                    // neither CTA leaves while the partner may still write to it or signal it
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
  if (threadIdx.x == 0 && *serr) atomicExch(gerr, 1);
}

template <int A_MN, int B_MN>
int launch_ksplit2(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const void* bias, int M, int N,
                   int K, int* gerr, cudaStream_t st) {
  auto kern = gemm_ksplit2_kernel<A_MN, B_MN>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_TOTAL);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int tiles = ((N + BN - 1) / BN) * ((M + BM - 1) / BM);
  kern<<<2 * tiles, NTHREADS, SMEM_TOTAL, st>>>(ta, tb, tc, (const bf16*)bias, M, N, K, gerr);
  DMB_CHECK_LAUNCH();
  return 0;
}

}  // namespace

extern "C" {

// Same contract as dmb_gemm_bf16 for bf16 results without accumulate (operand layouts, alignment, bias); refuses
// (-1) fp32 results, accumulate and reductions shorter than 8 k-blocks of 64.  One cluster of two CTAs per
// 128 x 256 tile: meant for at most (SMs / 2) tiles.
int dmb_gemm_bf16_ksplit2(const void* A, const void* B, void* C, const void* bias, int M, int N, int K, long long lda,
                          long long ldb, long long ldc, int a_mn, int b_mn, int out_f32, int accumulate, int* gerr,
                          cudaStream_t st) {
  if (!encode_fn()) return -10;
  if (N % 8 || out_f32 || accumulate || (a_mn && !b_mn) || K < 8 * BK) return -1;
  CUtensorMap ta, tb, tc;
  int rc;
  rc = a_mn ? make_map_2d(&ta, A, M, K, lda, 64, BK) : make_map_2d(&ta, A, K, M, lda, BK, BM);
  if (rc) return rc;
  rc = b_mn ? make_map_2d(&tb, B, N, K, ldb, 64, BK) : make_map_2d(&tb, B, K, N, ldb, BK, BN);
  if (rc) return rc;
  if ((rc = make_map_2d(&tc, C, N, M, ldc, 64, 32))) return rc;
  if (!a_mn && !b_mn) return launch_ksplit2<0, 0>(ta, tb, tc, bias, M, N, K, gerr, st);
  if (!a_mn && b_mn) return launch_ksplit2<0, 1>(ta, tb, tc, bias, M, N, K, gerr, st);
  return launch_ksplit2<1, 1>(ta, tb, tc, bias, M, N, K, gerr, st);
}

}  // extern "C"
