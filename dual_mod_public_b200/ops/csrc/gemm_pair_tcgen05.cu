// bf16 GEMM on CTA pairs: two CTAs of a cluster (two SMs) work on one 256 x BNP output tile (BNP = 256 or 128)
// with tcgen05.mma.cta_group::2.  Each CTA loads its own 128 rows of A and only HALF of the B tile (BNP / 2 of the
// BNP columns of C), so a k-block costs each SM 32 KB (BNP = 256) or 24 KB (BNP = 128) of shared-memory fill
// instead of 48 / 32 KB for a 128 x BNP tile of its own, and the tensor cores of both SMs read both halves.  The
// accumulator rows of a CTA (its 128 rows x BNP fp32 columns) live in that CTA's tensor memory and are written
// out by its own epilogue warps.  BNP = 128 is for problems with too few 256-wide tiles to fill the SMs (the
// input gradient of a sweep, 2048 x 1024 outputs over K = 4096): a CTA of its own on a 128 x 128 tile reads
// 8 KB of operands per 128 x 128 x 16 MMA from its shared memory, a CTA of a pair 6 KB.
//
//   C[M,N] (+)= op(A) . op(B)        same operand layouts and epilogues as the single-CTA kernel
//
// Roles per CTA: warp 0 = TMA producer (both CTAs load; every tile's bytes are counted on the LEADER's full
// barrier, the even CTA of the pair), warp 1 = tensor-memory owner and, in the leader only, MMA issuer,
// warps 2..5 = epilogue.  The leader's commits arrive on the barriers of both CTAs (one commit per CTA, no
// multicast); the epilogue warps of both CTAs arrive on the leader's accumulator-free barrier.  Persistent over
// tiles, shared-memory ring of 6 stages, accumulator double-buffered (2 x 256 columns = all of tensor memory).
// Every wait is bounded in time; on expiry the kernel raises the error flag, stops waiting and runs to its end
// (tensor memory released, the pair leaves together).
#include "tc05.cuh"

using namespace tc05;

namespace {

constexpr int BM = 128, BK = 64, UMMA_K = 16;
constexpr int A_BYTES = BM * BK * 2;
constexpr int NTHREADS = 192;

template <int BNP>
struct PairCfg {
  static constexpr int BN_HALF = BNP / 2;
  static constexpr int B_BYTES = BN_HALF * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = BNP == 256 ? 6 : 8;             // 192 KB of ring either way
  static constexpr int TMEM_COLS = 2 * BNP;                     // two accumulators
  static constexpr int stage_out_off = STAGES * STAGE_BYTES;    // epilogue staging: 4 warps x 2 slots x 4 KB
  static constexpr int bar_off = stage_out_off + 4 * 2 * 4096;
  static constexpr int SMEM_TOTAL = bar_off + 256;
};

// tile load whose completion bytes are counted on a barrier that may sit in the peer CTA of the pair
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar_cluster, int c0,
                                                 int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar_cluster), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void umma_pair_bf16(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc,
                                               uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrive on one barrier (a shared::cluster address: this CTA's or the peer's) when the pair's MMAs issued so far are done
__device__ __forceinline__ void umma_pair_commit(uint32_t bar_cluster) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster)
               : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(volatile uint32_t* slot, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)slot)), "r"(cols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t addr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}

template <int A_MN, int B_MN, int OUT_F32, int BNP>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NTHREADS, 1) gemm_pair_kernel(
    const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
    const __grid_constant__ CUtensorMap tmC, void* __restrict__ Cout, const bf16* __restrict__ bias, int M, int N,
    int K, long long ldc, int accumulate, int* __restrict__ gerr, int splits, float* __restrict__ ws) {
  using C = PairCfg<BNP>;
  constexpr int BN_PAIR = BNP, BN_HALF = C::BN_HALF, STAGES = C::STAGES, STAGE_BYTES = C::STAGE_BYTES;
  constexpr int TMEM_COLS = C::TMEM_COLS, stage_out_off = C::stage_out_off, bar_off = C::bar_off;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t base = smem_u32(smem_raw);
  uint8_t* base_ptr = smem_raw;
  const uint32_t bar0 = base + bar_off;
  // barriers (same offsets in both CTAs): full[s], empty[s], tmem_full[2], tmem_empty[2], TMEM address, error word
  auto full = [&](int s) { return bar0 + 8u * s; };
  auto empty = [&](int s) { return bar0 + 8u * (STAGES + s); };
  auto tmem_full = [&](int a) { return bar0 + 8u * (2 * STAGES + a); };
  auto tmem_empty = [&](int a) { return bar0 + 8u * (2 * STAGES + 2 + a); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(base_ptr + bar_off + 8 * (2 * STAGES + 4));
  volatile int* serr = reinterpret_cast<volatile int*>(base_ptr + bar_off + 8 * (2 * STAGES + 5));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();                    // 0 = leader
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const int tiles_n = (N + BN_PAIR - 1) / BN_PAIR, tiles_m = (M + 2 * BM - 1) / (2 * BM);
  const int KBT = (K + BK - 1) / BK, KBS = (KBT + splits - 1) / splits;
  const int n_items = tiles_n * tiles_m * splits;
  const bool aligned = (base & 1023u) == 0;

  if (threadIdx.x == 0) {
    *serr = aligned ? 0 : 1;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full(s), 1);             // the leader's own arrive.expect_tx; bytes of both CTAs
      mbar_init(empty(s), 1);            // one commit of the leader per use
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tmem_full(a), 1);
      mbar_init(tmem_empty(a), 8);       // four epilogue warps of each CTA (used in the leader only)
    }
    fence_barrier_init();
  }
  if (warp == 1) tmem_alloc_pair(tmem_slot, TMEM_COLS);
  tc_fence_before();
  cluster_sync_all();                    // the peer's barriers exist before anything arrives on them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------- TMA producer (both CTAs) ----------------
    if (lane == 0 && aligned) {
      uint32_t it = 0;
      bool alive = true;
      for (int item = pair; item < n_items && alive; item += n_pairs) {
        const int t2 = item / splits, ks = item - t2 * splits;
        const int m0 = (t2 / tiles_n) * 2 * BM + (int)rank * BM, n0 = (t2 % tiles_n) * BN_PAIR + (int)rank * BN_HALF;
        const int kb0 = ks * KBS, kb1 = min(KBT, kb0 + KBS);
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % STAGES;
          if (!mbar_wait(empty(s), ((it / STAGES) & 1) ^ 1, serr)) { alive = false; break; }
          const uint32_t sa = base + s * STAGE_BYTES, sb = sa + A_BYTES;
          if (rank == 0) mbar_expect_tx(full(s), 2 * STAGE_BYTES);
          const uint32_t lf = map_to_cta(full(s), 0);
          const int k0 = kb * BK;
          if (A_MN == 0) {
            tma_load_2d_pair(sa, &tmA, lf, k0, m0);                       // box {64 k, 128 m}
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_2d_pair(sa + j * (BK * 128), &tmA, lf, m0 + 64 * j, k0);
          }
          if (B_MN == 0) {
            tma_load_2d_pair(sb, &tmB, lf, k0, n0);                       // box {64 k, BNP / 2 n}
          } else {
#pragma unroll
            for (int j = 0; j < BN_HALF / 64; ++j) tma_load_2d_pair(sb + j * (BK * 128), &tmB, lf, n0 + 64 * j, k0);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (leader only) ----------------
    if (lane == 0 && rank == 0 && aligned) {
      constexpr uint32_t idesc = instr_desc(2 * BM, BN_PAIR, A_MN, B_MN);
      uint32_t it = 0, ti = 0;
      bool alive = true;
      for (int item = pair; item < n_items && alive; item += n_pairs, ++ti) {
        const uint32_t acc = ti & 1;
        if (!mbar_wait(tmem_empty(acc), ((ti >> 1) & 1) ^ 1, serr)) { alive = false; break; }
        tc_fence_after();
        const uint32_t tacc = tmem_base + acc * BN_PAIR;
        const int ks = item % splits, kb0 = ks * KBS, kb1 = min(KBT, kb0 + KBS);
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % STAGES;
          if (!mbar_wait(full(s), (it / STAGES) & 1, serr)) { alive = false; break; }
          tc_fence_after();
          const uint32_t sa = base + s * STAGE_BYTES, sb = sa + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t da = A_MN == 0 ? make_desc(sa + k * 32, 16, 1024) : make_desc(sa + k * 2048, BK * 128, 1024);
            const uint64_t db = B_MN == 0 ? make_desc(sb + k * 32, 16, 1024) : make_desc(sb + k * 2048, BK * 128, 1024);
            umma_pair_bf16(tacc, da, db, idesc, ((kb - kb0) | k) != 0);
          }
          umma_pair_commit(empty(s));                       // stage reusable in this CTA ...
          umma_pair_commit(map_to_cta(empty(s), 1));        // ... and in the peer
        }
        if (alive) {
          umma_pair_commit(tmem_full(acc));
          umma_pair_commit(map_to_cta(tmem_full(acc), 1));
        }
      }
    }
  } else {
    // ---------------- epilogue (both CTAs): this CTA's 128 rows x BNP columns ----------------
    const int q = warp & 3;
    uint32_t ti = 0, n_out = 0;
    bool alive = aligned;
    const uint32_t leader_empty0 = map_to_cta(tmem_empty(0), 0), leader_empty1 = map_to_cta(tmem_empty(1), 0);
    for (int item = pair; item < n_items && alive; item += n_pairs, ++ti) {
      const int t2 = item / splits, ks = item - t2 * splits;
      const int m0 = (t2 / tiles_n) * 2 * BM + (int)rank * BM, n0 = (t2 % tiles_n) * BN_PAIR;
      const uint32_t acc = ti & 1;
      if (!mbar_wait(tmem_full(acc), (ti >> 1) & 1, serr)) { alive = false; break; }
      tc_fence_after();
      const int row = m0 + q * 32 + lane;
      if (OUT_F32) {
#pragma unroll 1
        for (int c0 = 0; c0 < BN_PAIR; c0 += 32) {
          uint32_t r[32];
          tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN_PAIR + c0, r);
          tmem_ld_wait();
          const int col = n0 + c0;
          if (row < M && col < N) {
            float* dst = splits > 1 ? ws + ((long long)ks * M + row) * N + col
                                    : reinterpret_cast<float*>(Cout) + (long long)row * ldc + col;
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              if (col + j < N) {
                float4 v = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
                if (bias) {
                  v.x += __bfloat162float(bias[col + j]); v.y += __bfloat162float(bias[col + j + 1]);
                  v.z += __bfloat162float(bias[col + j + 2]); v.w += __bfloat162float(bias[col + j + 3]);
                }
                if (accumulate && splits == 1) {
                  float4 o = *reinterpret_cast<float4*>(dst + j);
                  v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
                }
                *reinterpret_cast<float4*>(dst + j) = v;
              }
            }
          }
        }
      } else {
        const bool rows_live = m0 + q * 32 < M;
#pragma unroll 1
        for (int c0 = 0; c0 < BN_PAIR; c0 += 64) {
          const int col = n0 + c0;
          if (col >= N) break;
          uint32_t r[64];
          {
            uint32_t (&ra)[32] = *reinterpret_cast<uint32_t (*)[32]>(&r[0]);
            uint32_t (&rb)[32] = *reinterpret_cast<uint32_t (*)[32]>(&r[32]);
            tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN_PAIR + c0, ra);
            tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN_PAIR + c0 + 32, rb);
          }
          tmem_ld_wait();
          if (!rows_live) continue;
          uint8_t* slot = base_ptr + stage_out_off + (q * 2 + (n_out & 1)) * 4096;
          if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
          __syncwarp();
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            float f[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              f[e] = __uint_as_float(r[j * 8 + e]);
              if (bias && col + j * 8 + e < N) f[e] += __bfloat162float(bias[col + j * 8 + e]);
            }
            const uint4 o = make_uint4(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]), pack_bf16(f[4], f[5]), pack_bf16(f[6], f[7]));
            *reinterpret_cast<uint4*>(slot + lane * 128 + ((j ^ (lane & 7)) << 4)) = o;
          }
          fence_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_2d(&tmC, smem_u32(slot), col, m0 + q * 32);
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          }
          ++n_out;
        }
      }
      // this warp has read its quarter of this CTA's accumulator: tell the leader's MMA issuer
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(acc ? leader_empty1 : leader_empty0);
    }
    if (!OUT_F32 && lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  }
  tc_fence_before();
  cluster_sync_all();                    // neither CTA leaves (or frees tensor memory) while the peer may still signal it
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
  if (threadIdx.x == 0 && *serr) atomicExch(gerr, 1);
}

// C[row, col] (+)= sum over slices of the split-K workspace (slices summed in index order)
__global__ void pair_splitk_reduce_kernel(float* __restrict__ Cout, const float* __restrict__ ws, int M, int N,
                                          long long ldc, int splits, int accumulate) {
  const long long n4 = (long long)M * N / 4;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    const long long e = i * 4, row = e / N, col = e - row * N;
    float4 a = *reinterpret_cast<const float4*>(ws + e);
    for (int s = 1; s < splits; ++s) {
      const float4 b = *reinterpret_cast<const float4*>(ws + (long long)s * M * N + e);
      a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
    }
    float* dst = Cout + row * ldc + col;
    if (accumulate) {
      const float4 o = *reinterpret_cast<const float4*>(dst);
      a.x += o.x; a.y += o.y; a.z += o.z; a.w += o.w;
    }
    *reinterpret_cast<float4*>(dst) = a;
  }
}

int g_pair_sms = 0;
int g_pair_bn = 0;                       // 0: chosen per problem; 128 / 256: forced (benchmarks, tests)
constexpr size_t PAIR_WS_BYTES = (size_t)64 << 20;
float* g_pair_ws[16] = {};

template <int A_MN, int B_MN, int OUT_F32, int BNP>
int launch_pair(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, void* C, const void* bias, int M,
                int N, int K, long long ldc, int accumulate, int* gerr, float* ws, int splits, cudaStream_t st) {
  auto kern = gemm_pair_kernel<A_MN, B_MN, OUT_F32, BNP>;
  constexpr int SMEM_TOTAL = PairCfg<BNP>::SMEM_TOTAL;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_TOTAL);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int tiles = ((N + BNP - 1) / BNP) * ((M + 2 * BM - 1) / (2 * BM));
  const int items = tiles * splits;
  const int pairs = items < g_pair_sms / 2 ? items : g_pair_sms / 2;
  kern<<<2 * pairs, NTHREADS, SMEM_TOTAL, st>>>(ta, tb, tc, C, (const bf16*)bias, M, N, K, ldc, accumulate, gerr, splits, ws);
  DMB_CHECK_LAUNCH();
  if (splits > 1) {
    pair_splitk_reduce_kernel<<<g_pair_sms * 2, 256, 0, st>>>((float*)C, ws, M, N, ldc, splits, accumulate);
    DMB_CHECK_LAUNCH();
  }
  return 0;
}

}  // namespace

extern "C" {

// forces the pair tile's width (128 or 256); 0 gives the choice back to the cost model
void dmb_gemm_pair_bn(int bn) { g_pair_bn = (bn == 128 || bn == 256) ? bn : 0; }

// Same contract as dmb_gemm_bf16 (operand layouts, alignment, epilogues); 256 x 256 or 256 x 128 tiles on CTA pairs.
int dmb_gemm_bf16_pair(const void* A, const void* B, void* C, const void* bias, int M, int N, int K, long long lda,
                       long long ldb, long long ldc, int a_mn, int b_mn, int out_f32, int accumulate, int* gerr,
                       cudaStream_t st) {
  if (!encode_fn()) return -10;
  if (N % 8 || (accumulate && !out_f32) || (a_mn && !b_mn)) return -1;
  if (!g_pair_sms) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&g_pair_sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || g_pair_sms < 2)
      return -12;
  }
  float* ws = nullptr;
  if (out_f32) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 16) return -12;
    if (!g_pair_ws[dev]) {
      cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
      cudaStreamIsCapturing(st, &cs);
      if (cs == cudaStreamCaptureStatusNone && cudaMalloc(&g_pair_ws[dev], PAIR_WS_BYTES) != cudaSuccess) g_pair_ws[dev] = nullptr;
    }
    ws = g_pair_ws[dev];
  }
  // Tile width and K split from a small cost model in units of one 256 x 256 x 64 k-block of a pair: a work item
  // costs kbs * a + e (a: k-block cost, e: epilogue), items run in ceil(items / pairs) rounds.  The K split is for
  // the weight-gradient shapes (few tiles, very long K; fp32 output only): work items of at least 16 k-blocks.
  int splits = 1, bnp = 256;
  {
    const int KBT = (K + BK - 1) / BK;
    const int pairs = g_pair_sms / 2;
    const long long tm = (M + 2 * BM - 1) / (2 * BM);
    double best = 1e30;
    for (int cand = 0; cand < 2; ++cand) {
      const int w = cand ? 128 : 256;
      if (g_pair_bn && w != g_pair_bn) continue;
      if (!g_pair_bn && N <= 128 && w == 256) continue;
      const long long tiles = (long long)((N + w - 1) / w) * tm;
      const double a = w == 256 ? 1.0 : 0.55, e = w == 256 ? 8.0 : 5.0;
      const int smax = (ws && !bias && N % 4 == 0 && tiles < pairs) ? 32 : 1;
      for (int sp = 1; sp <= smax; ++sp) {
        if (sp > 1 && (KBT / sp < 16 || (size_t)sp * M * N * sizeof(float) > PAIR_WS_BYTES)) break;
        const int kbs = (KBT + sp - 1) / sp;
        if (sp > 1 && (KBT + kbs - 1) / kbs != sp) continue;
        const long long rounds = (tiles * sp + pairs - 1) / pairs;
        double cost = rounds * (kbs * a + e);
        if (sp > 1) cost += (sp + 1.0) * M * N * 4.0 / 5e12 / 0.3e-6;
        if (cost < best) { best = cost; splits = sp; bnp = w; }
      }
    }
  }
  CUtensorMap ta, tb, tc;
  int rc;
  rc = a_mn ? make_map_2d(&ta, A, M, K, lda, 64, BK) : make_map_2d(&ta, A, K, M, lda, BK, BM);
  if (rc) return rc;
  rc = b_mn ? make_map_2d(&tb, B, N, K, ldb, 64, BK) : make_map_2d(&tb, B, K, N, ldb, BK, bnp / 2);
  if (rc) return rc;
  if (out_f32) tc = ta;
  else if ((rc = make_map_2d(&tc, C, N, M, ldc, 64, 32))) return rc;
#define GO(a, b, o)                                                                                                  \
  return bnp == 256 ? launch_pair<a, b, o, 256>(ta, tb, tc, C, bias, M, N, K, ldc, accumulate, gerr, ws, splits, st) \
                    : launch_pair<a, b, o, 128>(ta, tb, tc, C, bias, M, N, K, ldc, accumulate, gerr, ws, splits, st)
  if (!a_mn && !b_mn) { if (out_f32) GO(0, 0, 1); else GO(0, 0, 0); }
  if (!a_mn && b_mn) { if (out_f32) GO(0, 1, 1); else GO(0, 1, 0); }
  if (out_f32) GO(1, 1, 1); else GO(1, 1, 0);
#undef GO
}

}  // extern "C"
