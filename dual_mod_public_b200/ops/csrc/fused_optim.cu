// Data-parallel gradient reduction fused with the optimizer, over NVLink peer memory.
//
// Every rank holds the whole flat fp32 gradient buffer and the whole flat fp32 parameter buffer in
// peer-mapped memory, and the AdamW moments of the slices it owns.  The flat range is cut into
// buckets (one per layer, in the order the backward finishes them); inside a bucket rank r owns
// the r-th of `world` equal slices.  One cooperative kernel does, per rank:
//
//   phase 1  reduce-scatter: for every owned element, load it from every peer's gradient buffer
//            (plain P2P loads, fixed rank order => identical bytes everywhere), scale by
//            1/(world*accum), keep the fp32 result in the own buffer, and sum its square
//   phase 2  exchange the `world` partial squared norms through peer-mapped slots (bounded wait),
//            form the global norm, the clip coefficient and the skip predicate
//   phase 3  AdamW on the owned slices and all-gather: the updated fp32 parameter is stored
//            straight into every peer's parameter buffer (P2P stores)
//   phase 4  closing flag barrier: every rank's parameters are complete
//
// NVLS variant (DmbOptComm::mc_grads / mc_params set; the two buffers then come from an allocation bound to an
// NVLink multicast object): phase 1 is one multimem.ld_reduce.add per 16 bytes of the owned slice, the sum formed
// inside the switch (its order is the switch's, but only the owner reduces an element and everyone receives the
// owner's parameter, so all ranks still end with identical bytes); phase 3 is one multimem.st per 16 bytes.  Flags
// and norm slots stay on plain peer stores, every wait stays bounded.
//
// Buckets whose reduce-scatter already ran (launched early, overlapped with the backward, by
// dmb_opt_reduce_bucket) are skipped in phase 1.  Every cross-GPU wait is bounded in time; on
// expiry the kernel records where it gave up in `status` and carries on without hanging, the host
// reads the status word.  Peers are touched only by plain ld/st.global (no bulk-copy engine).
#include <cooperative_groups.h>
#include <string.h>

#include "common.cuh"

namespace cg = cooperative_groups;

#define DMB_MAX_WORLD 8
#define DMB_MAX_BUCKETS 64
#define DMB_MAX_SEGS 2048

struct DmbOptComm {
  int world, rank;
  float* grads[DMB_MAX_WORLD];         // peer-mapped flat gradient buffers
  float* params[DMB_MAX_WORLD];        // peer-mapped flat parameter buffers
  unsigned* flags[DMB_MAX_WORLD];      // peer-mapped flag pads: [n_slots][world]
  float* norms[DMB_MAX_WORLD];         // peer-mapped [2][world] partial squared norms (double buffered)
  // NVLink multicast addresses of the gradient and parameter buffers (NVLS), or null.  With them phase 1 reads
  // the sum over all ranks with one multimem.ld_reduce per 16 bytes (the switch adds) and phase 3 stores the
  // updated parameters to every rank with one multimem.st, instead of `world` peer loads / stores.
  float* mc_grads;
  float* mc_params;
};

struct DmbOptPlan {
  int n_buckets, n_segs;
  long long bucket_off[DMB_MAX_BUCKETS];   // element offset of the bucket in the flat buffer
  long long bucket_len[DMB_MAX_BUCKETS];   // elements, multiple of 4*world
  long long moment_off[DMB_MAX_BUCKETS];   // offset of this rank's slice in its m / v arrays
  int reduced[DMB_MAX_BUCKETS];            // 1: reduce-scatter already done for this bucket
};

struct DmbOptHyper {
  float lr, beta1, beta2, eps;
  float grad_scale;                            // 1 / (world * accum)
  float max_norm;                              // <= 0: no clipping
  float skip_norm;                             // > 0: skip the update when gnorm exceeds it
  unsigned epoch;                              // strictly increasing per launch
  long long wait_cycles;                       // bound of every cross-GPU wait, in clock64 ticks
};

// status word layout (host-visible): [0] error code (0 ok, 1 start barrier, 2 norm exchange,
// 3 end barrier), [1] peer that was missing, [2] skipped flag, [3] number of APPLIED updates so far
// (the AdamW step t: a skipped step does not advance it, as with torch.optim.AdamW when step() is
// not called)
// ctrl floats: [0] global grad norm, [1] clip coefficient, [2] skip (0/1), [3] spare (callers),
// [4] t, [5] 1 - beta1^t, [6] 1 - beta2^t, [7] the error code of status[0], so that one host copy of
// ctrl carries the verdict of the step and the health of the waits

namespace {

__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v));
}

// Threads 0..world-1 of one block: tell every peer "I reached `slot` at `epoch`", then wait until
// every peer said the same.  Returns the index of a missing peer, or -1.
__device__ int flag_barrier(const DmbOptComm& c, int slot, unsigned epoch, long long limit) {
  const int p = threadIdx.x;
  int missing = -1;
  if (p < c.world) {
    __threadfence_system();
    st_release_sys(c.flags[p] + slot * c.world + c.rank, epoch);
    const unsigned* mine = c.flags[c.rank] + slot * c.world + p;
    const long long t0 = clock64();
    while (ld_acquire_sys(mine) < epoch) {
      if (clock64() - t0 > limit) {
        missing = p;
        break;
      }
      __nanosleep(64);
    }
  }
  return missing;
}

__device__ __forceinline__ int find_seg(const long long* seg_start, int n, long long idx) {
  int lo = 0, hi = n - 1;
  while (lo < hi) {
    int mid = (lo + hi + 1) >> 1;
    if (seg_start[mid] <= idx) lo = mid; else hi = mid - 1;
  }
  return lo;
}

__device__ float block_sum(float v, float* sred) {
  v = warp_sum(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) sred[threadIdx.x >> 5] = v;
  __syncthreads();
  float s = 0.f;
  if (threadIdx.x < 32) {
    s = threadIdx.x < (blockDim.x >> 5) ? sred[threadIdx.x] : 0.f;
    s = warp_sum(s);
  }
  return s;  // valid in warp 0
}

// reduce-scatter of one bucket's owned slice; returns this thread's sum of squares
__device__ float reduce_slice(const DmbOptComm& c, long long off, long long len, float scale,
                              long long tid, long long nthreads) {
  const long long slice = len / c.world, base = off + (long long)c.rank * slice;
  float ss = 0.f;
  for (long long i = tid * 4; i < slice; i += nthreads * 4) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    if (c.mc_grads) {
      asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                   : "=f"(acc.x), "=f"(acc.y), "=f"(acc.z), "=f"(acc.w)
                   : "l"(c.mc_grads + base + i)
                   : "memory");
    } else {
      for (int p = 0; p < c.world; ++p) {
        float4 g = *reinterpret_cast<const float4*>(c.grads[p] + base + i);
        acc.x += g.x; acc.y += g.y; acc.z += g.z; acc.w += g.w;
      }
    }
    acc.x *= scale; acc.y *= scale; acc.z *= scale; acc.w *= scale;
    *reinterpret_cast<float4*>(c.grads[c.rank] + base + i) = acc;
    ss += acc.x * acc.x + acc.y * acc.y + acc.z * acc.z + acc.w * acc.w;
  }
  return ss;
}

__global__ void __launch_bounds__(512) reduce_bucket_kernel(DmbOptComm c, long long off, long long len,
                                                            float scale, float* __restrict__ partial,
                                                            unsigned epoch, int slot, long long limit,
                                                            unsigned* __restrict__ status) {
  __shared__ float sred[32];
  __shared__ int s_missing;
  // every block checks the peers itself (cheap: world flag reads) so no grid-wide sync is needed
  if (threadIdx.x == 0) s_missing = -1;
  __syncthreads();
  if (threadIdx.x < c.world) {
    const unsigned* mine = c.flags[c.rank] + slot * c.world + threadIdx.x;
    const long long t0 = clock64();
    while (ld_acquire_sys(mine) < epoch) {
      if (clock64() - t0 > limit) { s_missing = threadIdx.x; break; }
      __nanosleep(64);
    }
  }
  __syncthreads();
  if (s_missing >= 0) {
    if (threadIdx.x == 0) { status[0] = 1; status[1] = s_missing; }
    if (threadIdx.x == 0) partial[blockIdx.x] = 0.f;
    return;
  }
  float ss = reduce_slice(c, off, len, scale, (long long)blockIdx.x * blockDim.x + threadIdx.x,
                          (long long)gridDim.x * blockDim.x);
  ss = block_sum(ss, sred);
  if (threadIdx.x == 0) partial[blockIdx.x] = ss;
}

// "my gradients for this bucket are final": one flag store per peer
__global__ void signal_kernel(DmbOptComm c, int slot, unsigned epoch) {
  if (threadIdx.x < c.world) {
    __threadfence_system();
    st_release_sys(c.flags[threadIdx.x] + slot * c.world + c.rank, epoch);
  }
}

__global__ void __launch_bounds__(512) fused_step_kernel(
    DmbOptComm c, DmbOptPlan plan, DmbOptHyper hp, const long long* __restrict__ seg_start,
    const float* __restrict__ seg_wd, const float* __restrict__ seg_lr, float* __restrict__ m,
    float* __restrict__ v, float* __restrict__ partial /* [gridDim.x + early partials] */,
    int n_early_partials, float* __restrict__ ctrl, unsigned* __restrict__ status) {
  cg::grid_group grid = cg::this_grid();
  __shared__ float sred[32];
  __shared__ float s_coef, s_skip, s_bias1, s_bias2;
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long nthreads = (long long)gridDim.x * blockDim.x;

  // ---- opening barrier: all ranks' gradients are final ----------------------------------------
  if (blockIdx.x == 0) {
    int miss = flag_barrier(c, 0, hp.epoch, hp.wait_cycles);
    if (miss >= 0) { status[0] = 1; status[1] = miss; }
  }
  grid.sync();

  // ---- phase 1: reduce-scatter (+ scale, + sum of squares) --------------------------------------
  float ss = 0.f;
  for (int b = 0; b < plan.n_buckets; ++b)
    if (!plan.reduced[b]) ss += reduce_slice(c, plan.bucket_off[b], plan.bucket_len[b], hp.grad_scale, tid, nthreads);
  ss = block_sum(ss, sred);
  if (threadIdx.x == 0) partial[n_early_partials + blockIdx.x] = ss;
  grid.sync();

  // ---- phase 2: global norm over ranks, clip coefficient, skip predicate -------------------------
  if (blockIdx.x == 0) {
    float loc = 0.f;
    const int n_part = n_early_partials + gridDim.x;
    for (int i = threadIdx.x; i < n_part; i += blockDim.x) loc += partial[i];
    loc = block_sum(loc, sred);
    const int buf = hp.epoch & 1;
    if (threadIdx.x == 0) {
      for (int p = 0; p < c.world; ++p) c.norms[p][buf * c.world + c.rank] = loc;
    }
    __syncthreads();
    int miss = flag_barrier(c, 1, hp.epoch, hp.wait_cycles);
    if (miss >= 0) { status[0] = 2; status[1] = miss; }
    __syncthreads();
    if (threadIdx.x == 0) {
      float tot = 0.f;
      for (int p = 0; p < c.world; ++p) tot += c.norms[c.rank][buf * c.world + p];
      const float gn = sqrtf(tot);
      float coef = 1.f;
      if (hp.max_norm > 0.f) coef = fminf(1.f, hp.max_norm / (gn + 1e-6f));
      const bool skip = !isfinite(gn) || (hp.skip_norm > 0.f && gn > hp.skip_norm) || status[0] != 0;
      ctrl[0] = gn; ctrl[1] = coef; ctrl[2] = skip ? 1.f : 0.f;
      status[2] = skip ? 1u : 0u;
      unsigned t = status[3];
      if (!skip) status[3] = ++t;
      const double td = t ? (double)t : 1.0;
      ctrl[4] = (float)t;
      ctrl[5] = (float)(1.0 - pow((double)hp.beta1, td));
      ctrl[6] = (float)(1.0 - pow((double)hp.beta2, td));
      ctrl[7] = (float)status[0];
      __threadfence();
    }
  }
  grid.sync();
  if (threadIdx.x == 0) { s_coef = ctrl[1]; s_skip = ctrl[2]; s_bias1 = ctrl[5]; s_bias2 = ctrl[6]; }
  __syncthreads();
  const float coef = s_coef;

  // ---- phase 3: AdamW on the owned slices + all-gather by peer stores -----------------------------
  if (s_skip == 0.f) {
    const float step_size = hp.lr / s_bias1, inv_sqrt_b2 = rsqrtf(s_bias2);
    for (int b = 0; b < plan.n_buckets; ++b) {
      const long long slice = plan.bucket_len[b] / c.world;
      const long long base = plan.bucket_off[b] + (long long)c.rank * slice, mo = plan.moment_off[b];
      // one binary search per thread and bucket; after it the thread's index only grows, so the
      // parameter it falls into is found by walking forward (a float4 never straddles two parameters:
      // every parameter starts on a 64-element boundary)
      int sg = tid * 4 < slice ? find_seg(seg_start, plan.n_segs, base + tid * 4) : 0;
      for (long long i = tid * 4; i < slice; i += nthreads * 4) {
        while (sg + 1 < plan.n_segs && seg_start[sg + 1] <= base + i) ++sg;
        const float wd = seg_wd[sg], lrm = seg_lr[sg];
        float4 g = *reinterpret_cast<const float4*>(c.grads[c.rank] + base + i);
        float4 p = *reinterpret_cast<const float4*>(c.params[c.rank] + base + i);
        float4 mm = *reinterpret_cast<const float4*>(m + mo + i);
        float4 vv = *reinterpret_cast<const float4*>(v + mo + i);
        float* gp = &g.x; float* pp = &p.x; float* mp = &mm.x; float* vp = &vv.x;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float ge = gp[e] * coef;
          mp[e] = hp.beta1 * mp[e] + (1.f - hp.beta1) * ge;
          vp[e] = hp.beta2 * vp[e] + (1.f - hp.beta2) * ge * ge;
          const float denom = sqrtf(vp[e]) * inv_sqrt_b2 + hp.eps;
          pp[e] = pp[e] * (1.f - hp.lr * lrm * wd) - step_size * lrm * mp[e] / denom;
        }
        *reinterpret_cast<float4*>(m + mo + i) = mm;
        *reinterpret_cast<float4*>(v + mo + i) = vv;
        if (c.mc_params) {
          asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};"
                       ::"l"(c.mc_params + base + i), "f"(p.x), "f"(p.y), "f"(p.z), "f"(p.w)
                       : "memory");
        } else {
          for (int q = 0; q < c.world; ++q) {
            const int peer = (c.rank + q) % c.world;      // spread the store targets over the links
            *reinterpret_cast<float4*>(c.params[peer] + base + i) = p;
          }
        }
      }
    }
  }
  __threadfence_system();
  grid.sync();

  // ---- closing barrier: everybody's parameter stores have landed ----------------------------------
  if (blockIdx.x == 0) {
    int miss = flag_barrier(c, 2, hp.epoch, hp.wait_cycles);
    if (miss >= 0 && status[0] == 0) { status[0] = 3; status[1] = miss; }
    __syncthreads();
    if (threadIdx.x == 0) ctrl[7] = (float)status[0];
  }
}

}  // namespace

extern "C" {

// ---- peer-memory plumbing (CUDA IPC; one process per GPU on one node) -----------------------------
int dmb_ipc_alloc(size_t bytes, void** ptr) {
  cudaError_t e = cudaMalloc(ptr, bytes);
  if (e != cudaSuccess) return (int)e;
  return (int)cudaMemset(*ptr, 0, bytes);
}
int dmb_ipc_free(void* ptr) { return (int)cudaFree(ptr); }
int dmb_ipc_get_handle(void* ptr, void* out64) {
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, ptr);
  if (e != cudaSuccess) return (int)e;
  memcpy(out64, &h, sizeof(h));
  return 0;
}
int dmb_ipc_open(const void* in64, void** ptr) {
  cudaIpcMemHandle_t h;
  memcpy(&h, in64, sizeof(h));
  return (int)cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess);
}
int dmb_ipc_close(void* ptr) { return (int)cudaIpcCloseMemHandle(ptr); }
int dmb_ipc_handle_size() { return (int)sizeof(cudaIpcMemHandle_t); }

int dmb_opt_struct_sizes(int* comm, int* plan, int* hyper) {
  *comm = (int)sizeof(DmbOptComm);
  *plan = (int)sizeof(DmbOptPlan);
  *hyper = (int)sizeof(DmbOptHyper);
  return 0;
}

int dmb_opt_signal(const DmbOptComm* c, int slot, unsigned epoch, cudaStream_t st) {
  signal_kernel<<<1, 32, 0, st>>>(*c, slot, epoch);
  DMB_CHECK_LAUNCH();
  return 0;
}

// early reduce-scatter of one bucket (overlaps the rest of the backward).  `partial` receives
// `blocks` floats.  `slot` is the per-bucket readiness flag row signalled by dmb_opt_signal.
int dmb_opt_reduce_bucket(const DmbOptComm* c, long long off, long long len, float scale,
                          float* partial, int blocks, unsigned epoch, int slot, long long wait_cycles,
                          unsigned* status, cudaStream_t st) {
  reduce_bucket_kernel<<<blocks, 512, 0, st>>>(*c, off, len, scale, partial, epoch, slot, wait_cycles, status);
  DMB_CHECK_LAUNCH();
  return 0;
}

int dmb_opt_max_blocks(int* out) {
  int dev, sms, per_sm;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (e != cudaSuccess) return (int)e;
  e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fused_step_kernel, 512, 0);
  if (e != cudaSuccess) return (int)e;
  *out = sms * (per_sm > 2 ? 2 : per_sm);
  return 0;
}

int dmb_opt_fused_step(const DmbOptComm* c, const DmbOptPlan* plan, const DmbOptHyper* hp,
                       const long long* seg_start, const float* seg_wd, const float* seg_lr, float* m,
                       float* v, float* partial, int n_early_partials, float* ctrl, unsigned* status,
                       int blocks, cudaStream_t st) {
  DmbOptComm cc = *c;
  DmbOptPlan pp = *plan;
  DmbOptHyper hh = *hp;
  void* args[] = {&cc, &pp, &hh, &seg_start, &seg_wd, &seg_lr, &m, &v, &partial, &n_early_partials, &ctrl, &status};
  cudaError_t e = cudaLaunchCooperativeKernel((void*)fused_step_kernel, dim3(blocks), dim3(512), args, 0, st);
  return (int)e;
}

}  // extern "C"
