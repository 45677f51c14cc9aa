// bf16 GEMM on the 5th-generation tensor cores: TMA-fed shared-memory pipeline, tcgen05.mma issued
// by one elected thread, fp32 accumulator in tensor memory, epilogue read back with tcgen05.ld.
//
//   C[M,N] (+)= op(A) . op(B)        fp32 accumulate, C stored as bf16 or fp32
//
// Operand layouts (both bf16, innermost dimension contiguous):
//   A_MN = 0 : A stored [M][K]  (K-major)        A_MN = 1 : A stored [K][M]  (M-major)
//   B_MN = 0 : B stored [N][K]  (K-major)        B_MN = 1 : B stored [K][N]  (N-major)
// which covers y = x W^T (0,0), dx = dy W (0,1) and dW += dy^T x (1,1) without any transpose pass.
//
// Persistent kernel, one CTA per SM, 128 x BN output tiles (BN = 256, or 128 for narrow problems)
// handed out round-robin.  warp 0 = TMA producer, warp 1 = MMA issuer (+ TMEM owner), warps 2..5 =
// epilogue (each reads its own 32-lane quarter of TMEM).  The shared-memory ring of 128B-swizzled
// tiles runs on across tile boundaries, and the accumulator is double-buffered in TMEM (2 x BN
// columns), so the epilogue of tile i overlaps the main loop of tile i+1.  Each CTA
// loads its own tiles.  Every mbarrier wait is bounded in time: on expiry the kernel raises a flag in global
// memory, stops waiting and runs to its end so TMEM is released.
#include "tc05.cuh"

using namespace tc05;

namespace {

constexpr int BM = 128, BK = 64, UMMA_K = 16;
constexpr int A_BYTES = BM * BK * 2;
constexpr int NTHREADS = 192;

template <int BN>
struct Cfg {
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = BN == 256 ? 4 : 6;
  static constexpr int TMEM_COLS = 2 * BN;              // two accumulators
  static constexpr int stage_out_off = STAGES * STAGE_BYTES;      // epilogue staging: 4 warps x 2 slots x 4 KB
  static constexpr int bar_off = stage_out_off + 4 * 2 * 4096;    // tiles first (1024-byte aligned base), barriers after
  static constexpr int total = bar_off + 256;
};
template <int A_MN, int B_MN, int OUT_F32, int BN>
__global__ void __launch_bounds__(NTHREADS, 1) gemm_kernel(
    const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
    const __grid_constant__ CUtensorMap tmC, void* __restrict__ Cout,
    const bf16* __restrict__ bias, int M, int N, int K, long long ldc, int accumulate, int* __restrict__ gerr,
    int splits, float* __restrict__ ws) {
  using C = Cfg<BN>;
  constexpr int STAGES = C::STAGES, STAGE_BYTES = C::STAGE_BYTES;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t bar0 = base + C::bar_off;
  // barriers: full[s], empty[s], tmem_full[2], tmem_empty[2], then the TMEM address slot and the error word
  auto full = [&](int s) { return bar0 + 8u * s; };
  auto empty = [&](int s) { return bar0 + 8u * (STAGES + s); };
  auto tmem_full = [&](int a) { return bar0 + 8u * (2 * STAGES + a); };
  auto tmem_empty = [&](int a) { return bar0 + 8u * (2 * STAGES + 2 + a); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(base_ptr + C::bar_off + 8 * (2 * STAGES + 4));
  volatile int* serr = reinterpret_cast<volatile int*>(base_ptr + C::bar_off + 8 * (2 * STAGES + 5));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_n = (N + BN - 1) / BN, tiles_m = (M + BM - 1) / BM;
  // split-K: work item w = tile * splits + ks covers k-blocks [ks * KBS, min(KBT, (ks + 1) * KBS)) and
  // writes its partial product to slice ks of the fp32 workspace; a second kernel sums the slices
  const int KBT = (K + BK - 1) / BK, KBS = (KBT + splits - 1) / splits;
  const int n_tiles = tiles_n * tiles_m * splits;

  if (threadIdx.x == 0) {
    *serr = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full(s), 1);
      mbar_init(empty(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tmem_full(a), 1);
      mbar_init(tmem_empty(a), 4);       // one arrival per epilogue warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, C::TMEM_COLS);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------- TMA producer: the ring position `it` runs on across tiles ----------------
    if (lane == 0) {
      uint32_t it = 0;
      bool alive = true;
      for (int tile = blockIdx.x; tile < n_tiles && alive; tile += gridDim.x) {
        const int t2 = tile / splits, ks = tile - t2 * splits;
        const int m0 = (t2 / tiles_n) * BM, n0 = (t2 % tiles_n) * BN;
        const int kb0 = ks * KBS, kb1 = min(KBT, kb0 + KBS);
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % STAGES;
          if (!mbar_wait(empty(s), ((it / STAGES) & 1) ^ 1, serr)) { alive = false; break; }
          const uint32_t sa = base + s * STAGE_BYTES, sb = sa + A_BYTES;
          mbar_expect_tx(full(s), STAGE_BYTES);
          const int k0 = kb * BK;
          if (A_MN == 0) {
            tma_load_2d(sa, &tmA, full(s), k0, m0);                       // box {64 k, 128 m}
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_2d(sa + j * (BK * 128), &tmA, full(s), m0 + 64 * j, k0);  // box {64 m, 64 k}
          }
          if (B_MN == 0) {
            tma_load_2d(sb, &tmB, full(s), k0, n0);                       // box {64 k, BN n}
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) tma_load_2d(sb + j * (BK * 128), &tmB, full(s), n0 + 64 * j, k0);  // box {64 n, 64 k}
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idesc = instr_desc(BM, BN, A_MN, B_MN);
      uint32_t it = 0, ti = 0;
      bool alive = true;
      for (int tile = blockIdx.x; tile < n_tiles && alive; tile += gridDim.x, ++ti) {
        const uint32_t acc = ti & 1;
        // the epilogue must have drained this accumulator (two tiles ago)
        if (!mbar_wait(tmem_empty(acc), ((ti >> 1) & 1) ^ 1, serr)) { alive = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t tacc = tmem_base + acc * BN;
        const int ks = tile % splits, kb0 = ks * KBS, kb1 = min(KBT, kb0 + KBS);
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % STAGES;
          if (!mbar_wait(full(s), (it / STAGES) & 1, serr)) { alive = false; break; }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t sa = base + s * STAGE_BYTES, sb = sa + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            // K-major: 32 bytes further along the swizzled 128-byte row; MN-major: 16 k-rows of 128 bytes
            const uint64_t da = A_MN == 0 ? make_desc(sa + k * 32, 16, 1024) : make_desc(sa + k * 2048, BK * 128, 1024);
            const uint64_t db = B_MN == 0 ? make_desc(sb + k * 32, 16, 1024) : make_desc(sb + k * 2048, BK * 128, 1024);
            umma_bf16(tacc, da, db, idesc, ((kb - kb0) | k) != 0);
          }
          umma_commit(empty(s));           // stage reusable once these MMAs have read it
        }
        if (alive) umma_commit(tmem_full(acc));   // accumulator complete
      }
    }
  } else {
    // ---------------- epilogue: TMEM -> registers -> global ----------------
    const int q = warp & 3;              // TMEM lane quarter this warp may touch
    uint32_t ti = 0, n_out = 0;          // n_out: staging slots handed to TMA stores so far (parity picks the slot)
    bool alive = true;
    for (int tile = blockIdx.x; tile < n_tiles && alive; tile += gridDim.x, ++ti) {
      const int t2 = tile / splits, ks = tile - t2 * splits;
      const int m0 = (t2 / tiles_n) * BM, n0 = (t2 % tiles_n) * BN;
      const uint32_t acc = ti & 1;
      if (!mbar_wait(tmem_full(acc), (ti >> 1) & 1, serr)) { alive = false; break; }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int row = m0 + q * 32 + lane;
      if (OUT_F32) {
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 32) {
          uint32_t r[32];
          tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN + c0, r);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          const int col = n0 + c0;
          if (row < M && col < N) {
            float* dst = splits > 1 ? ws + ((long long)ks * M + row) * N + col
                                    : reinterpret_cast<float*>(Cout) + (long long)row * ldc + col;
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              if (col + j < N) {      // N % 8 == 0 keeps groups of 4 whole
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
        // bf16: 64 columns at a time through this warp's two staging slots
        const bool rows_live = m0 + q * 32 < M;           // warp-uniform
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 64) {
          const int col = n0 + c0;
          if (col >= N) break;                             // warp-uniform: the rest of the tile is outside C
          uint32_t r[64];
          {
            uint32_t (&ra)[32] = *reinterpret_cast<uint32_t (*)[32]>(&r[0]);
            uint32_t (&rb)[32] = *reinterpret_cast<uint32_t (*)[32]>(&r[32]);
            tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN + c0, ra);
            tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN + c0 + 32, rb);
          }
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          if (!rows_live) continue;
          uint8_t* slot = base_ptr + C::stage_out_off + (q * 2 + (n_out & 1)) * 4096;
          // the store that last read this slot (two chunks ago) must have drained it
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
            // 128-byte swizzle: 16-byte chunk j of row `lane` sits at chunk j ^ (lane & 7)
            *reinterpret_cast<uint4*>(slot + lane * 128 + ((j ^ (lane & 7)) << 4)) = o;
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          __syncwarp();
          if (lane == 0) {
            tma_store_2d(&tmC, smem_u32(slot), col, m0 + q * 32);
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          }
          ++n_out;
        }
      }
      // this warp has read its quarter of the accumulator: hand it back to the MMA issuer
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(tmem_empty(acc));
    }
    if (!OUT_F32 && lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");   // stores complete before exit
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
  if (threadIdx.x == 0 && *serr) atomicExch(gerr, 1);
}

// C[row, col] (+)= sum over slices of the split-K workspace (slices summed in index order)
__global__ void splitk_reduce_kernel(float* __restrict__ Cout, const float* __restrict__ ws, int M, int N, long long ldc,
                                     int splits, int accumulate) {
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

int g_sms = 0;
constexpr size_t WS_BYTES = (size_t)64 << 20;    // split-K workspace, one per device, allocated on first use
float* g_ws[16] = {};

template <int A_MN, int B_MN, int OUT_F32, int BN>
int launch(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, void* C, const void* bias, int M, int N, int K,
           long long ldc, int accumulate, int* gerr, float* ws, int splits, cudaStream_t st) {
  auto kern = gemm_kernel<A_MN, B_MN, OUT_F32, BN>;
  static bool configured = false;
  const int smem = Cfg<BN>::total + 1024;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int tiles = ((N + BN - 1) / BN) * ((M + BM - 1) / BM);
  const int items = tiles * splits;
  kern<<<items < g_sms ? items : g_sms, NTHREADS, smem, st>>>(ta, tb, tc, C, (const bf16*)bias, M, N, K, ldc, accumulate,
                                                             gerr, splits, ws);
  DMB_CHECK_LAUNCH();
  if (splits > 1) {
    splitk_reduce_kernel<<<g_sms * 2, 256, 0, st>>>((float*)C, ws, M, N, ldc, splits, accumulate);
    DMB_CHECK_LAUNCH();
  }
  return 0;
}

}  // namespace

extern "C" {

// C[M,N] (+)= op(A) op(B).  lda / ldb: row stride (elements) of A and B as stored.
//   a_mn = 0: A stored [M][K];  a_mn = 1: A stored [K][M]      (same for B with N)
// Supported layouts: (0,0) y = x W^T, (0,1) dx = dy W, (1,1) dW += dy^T x.
// Requirements: pointers 16-byte aligned, lda/ldb/ldc multiples of 8 (bf16) resp. 4 (fp32 C),
// N % 8 == 0.  out_f32: C is fp32 (else bf16).  accumulate needs out_f32.  `gerr` (device int) is
// set to 1 if a pipeline wait ran out.
int dmb_gemm_bf16(const void* A, const void* B, void* C, const void* bias, int M, int N, int K, long long lda,
                  long long ldb, long long ldc, int a_mn, int b_mn, int out_f32, int accumulate, int* gerr,
                  cudaStream_t st) {
  if (!encode_fn()) return -10;
  if (N % 8 || (accumulate && !out_f32) || (a_mn && !b_mn)) return -1;
  if (!g_sms) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&g_sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || g_sms <= 0)
      return -12;
  }
  float* ws = nullptr;
  if (out_f32) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 16) return -12;
    if (!g_ws[dev]) {
      cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
      cudaStreamIsCapturing(st, &cs);
      if (cs == cudaStreamCaptureStatusNone && cudaMalloc(&g_ws[dev], WS_BYTES) != cudaSuccess) g_ws[dev] = nullptr;
    }
    ws = g_ws[dev];                                  // null: no split-K (allocation failed or capturing)
  }
  // tile width and K split from a small cost model, in units of one 128x256x64 k-block: a work item
  // costs kbs * a + e (a: k-block cost, e: epilogue), items run in ceil(items / SMs) rounds, and a
  // split adds the workspace round trip.  Splitting is for the weight-gradient shapes (small M x N,
  // very long K) and needs the fp32 output path.
  int bn = 256, splits = 1;
  {
    const int KBT = (K + BK - 1) / BK;
    const int tm = (M + BM - 1) / BM;
    double best = 1e30;
    for (int cand = 0; cand < 2; ++cand) {
      const int w = cand ? 128 : 256;
      if (N <= 128 && w == 256) continue;
      const long long tiles = (long long)((N + w - 1) / w) * tm;
      const double a = w == 256 ? 1.0 : 0.6, e = w == 256 ? 8.0 : 4.0;
      const int smax = (ws && !bias && N % 4 == 0) ? 16 : 1;
      for (int sp = 1; sp <= smax; ++sp) {
        if (sp > 1 && (KBT / sp < 16 || (size_t)sp * M * N * sizeof(float) > WS_BYTES)) break;
        const int kbs = (KBT + sp - 1) / sp;
        if (sp > 1 && (KBT + kbs - 1) / kbs != sp) continue;          // would leave an empty slice
        const long long rounds = (tiles * sp + g_sms - 1) / g_sms;
        double cost = rounds * (kbs * a + e);
        if (sp > 1) cost += (sp + 1.0) * M * N * 4.0 / 5e12 / 0.41e-6;
        if (cost < best) { best = cost; bn = w; splits = sp; }
      }
    }
  }
  CUtensorMap ta, tb, tc;
  int rc;
  rc = a_mn ? make_map_2d(&ta, A, M, K, lda, 64, BK) : make_map_2d(&ta, A, K, M, lda, BK, BM);
  if (rc) return rc;
  rc = b_mn ? make_map_2d(&tb, B, N, K, ldb, 64, BK) : make_map_2d(&tb, B, K, N, ldb, BK, bn);
  if (rc) return rc;
  // bf16 results leave through TMA stores of 32-row x 64-column boxes (fp32 results are stored directly)
  if (out_f32) tc = ta;
  else if ((rc = make_map_2d(&tc, C, N, M, ldc, 64, 32))) return rc;
#define GO(a, b, o)                                                                               \
  return bn == 256 ? launch<a, b, o, 256>(ta, tb, tc, C, bias, M, N, K, ldc, accumulate, gerr, ws, splits, st)    \
                   : launch<a, b, o, 128>(ta, tb, tc, C, bias, M, N, K, ldc, accumulate, gerr, ws, splits, st)
  if (!a_mn && !b_mn) { if (out_f32) GO(0, 0, 1); else GO(0, 0, 0); }
  if (!a_mn && b_mn) { if (out_f32) GO(0, 1, 1); else GO(0, 1, 0); }
  if (out_f32) GO(1, 1, 1); else GO(1, 1, 0);
#undef GO
}

}  // extern "C"
