// Collectives written as kernels over peer-mapped (symmetric) memory on one NVSwitch box.
//
//  * gf_signal_peers / gf_wait_flags : system-scope release/acquire flags in each rank's signal pad.
//  * gf_rs_adamw_fused : gradient reduce-scatter fused with the sharded AdamW update. Each rank reads its
//      slice of EVERY rank's bf16 gradient buffer straight over NVLink (plain peer loads, or one
//      multimem.ld_reduce through the switch when a multicast mapping is given), sums in fp32, and
//      applies AdamW to its fp32 master/moment shard, writing the bf16 weight shard in the same pass.
//      The reduced gradient never exists in memory.
//  * gf_allgather_pull : parameter all-gather; each rank copies the peers' bf16 shards into its local
//      gathered buffer and raises one local flag per source shard, which the GEMM producer
//      (gemm_bf16.cu, b_ready) can wait on tile by tile.
//
// Every wait is bounded and reports through the status word; nothing here uses TMA, let alone
// cluster multicast, on peer memory.
//
// The reference only simulates these collectives in-process (reduce-scatter = divide by world size,
// all-gather = clone: ghostflow-nn/src/zero_optimizer.rs:220-259) and its optimizer step has no bias
// correction or weight decay (zero_optimizer.rs:262-309); the update here is the AdamW of
// ghostflow-optim/src/adam.rs:162-197.
#include "gf_host.h"
#include "gf_ptx.cuh"

namespace gf {

constexpr int MAX_RANKS = 8;

struct PeerPtrs {
  const void* p[MAX_RANKS];
};
struct PeerFlagPtrs {
  int* p[MAX_RANKS];
};

__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_release_gpu(int* p, int v) {
  asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Bounded wait until *flag >= value. Returns false when the limit ran out.
__device__ __forceinline__ bool wait_flag_ge(const int* flag, int value, uint32_t limit) {
  for (uint32_t it = 0; it < limit; ++it) {
    if (ld_acquire_sys(flag) >= value) return true;
    __nanosleep(100);
  }
  return false;
}

// ------------------------------------------------------------------ flags
// Thread r writes `value` into rank r's pad at index idx_base + my_rank.
// `epoch` (may be null) points to a device counter whose value is added to the flag value: launches recorded
// once in a CUDA graph then publish / expect a new value on every replay.
__global__ void signal_peers_kernel(PeerFlagPtrs pads, int idx_base, int my_rank, int world, int value,
                                    const int* epoch) {
  const int r = threadIdx.x;
  if (epoch) value += *epoch;
  if (r < world) {
    __threadfence_system();
    st_release_sys(pads.p[r] + idx_base + my_rank, value);
  }
}

// Thread r waits for local_pad[idx_base + r] >= value.
__global__ void wait_flags_kernel(const int* local_pad, int idx_base, int world, int value, uint32_t limit,
                                  int* status, const int* epoch) {
  const int r = threadIdx.x;
  if (epoch) value += *epoch;
  if (r < world) {
    if (!wait_flag_ge(local_pad + idx_base + r, value, limit) && status) atomicCAS(status, 0, GF_ERR_WAIT_PEER);
  }
}

// ------------------------------------------------------------------ reduce-scatter + AdamW
struct RsAdamArgs {
  PeerPtrs grads;           // each rank's full bf16 gradient buffer (same layout everywhere)
  const void* mc_grads;     // multicast mapping of the same buffer, or null
  long long shard_lo;       // first element of this rank's shard inside the full buffer
  long long n;              // shard elements (multiple of 8)
  float* master;
  float* m;
  float* v;
  __nv_bfloat16* p_lp;      // bf16 weight shard (may be null)
  float lr, beta1, beta2, eps, wd, bc1, bc2, grad_scale;
  int world, my_rank;
  // flags
  const int* local_pad;     // this rank's pad
  PeerFlagPtrs pads;        // every rank's pad
  int ready_idx;            // wait: local_pad[ready_idx + r] >= ready_val for all r
  int ready_val;
  int consumed_idx;         // afterwards: pads[r][consumed_idx + my_rank] = consumed_val
  int consumed_val;
  int version_idx;          // afterwards: pads[r][version_idx + my_rank] = version_val (weights updated)
  int version_val;
  int* done_counter;        // local int, zero before launch; reset by the last block
  uint32_t wait_limit;
  int* status;
  // reduce-only mode (gradient clipping / overflow check need the global norm before any update): the reduced,
  // scaled gradient of the shard goes to grad_out (fp32) and its sum of squares is added to *sumsq; master, moments
  // and weights are left alone and no version flag is published
  float* grad_out;
  float* sumsq;
  // optional device counter (graph replays): added to ready_val / consumed_val / version_val, and, when
  // step_from_epoch is set, the bias corrections are computed from it (Adam step = *epoch)
  const int* epoch;
  int step_from_epoch;
};

// Register budget: at most 64 per thread (4 CTAs of 256 threads per SM) and one CTA per SM in the launch, so
// that the persistent GEMM / all-gather CTAs of the other streams always find room beside it. With a larger
// footprint those kernels cannot start until this one has drained, and the "overlapped" update serialises.
template <bool USE_MC, bool REDUCE_ONLY = false>
__global__ void __launch_bounds__(256, 4)
rs_adamw_kernel(const RsAdamArgs a) {
  __shared__ int s_ok;
  __shared__ float s_sq[8];
  float sq = 0.f;
  const int ep = a.epoch ? *a.epoch : 0;
  float bc1 = a.bc1, bc2 = a.bc2;
  if (a.step_from_epoch) {
    bc1 = 1.f - powf(a.beta1, (float)ep);
    bc2 = 1.f - powf(a.beta2, (float)ep);
  }
  if (threadIdx.x < 32) {
    bool ok = true;
    if (threadIdx.x < a.world)
      ok = wait_flag_ge(a.local_pad + a.ready_idx + threadIdx.x, a.ready_val + ep, a.wait_limit);
    ok = __all_sync(0xffffffffu, ok);
    if (threadIdx.x == 0) {
      s_ok = ok ? 1 : 0;
      if (!ok && a.status) atomicCAS(a.status, 0, GF_ERR_WAIT_PEER);
    }
  }
  __syncthreads();
  if (s_ok) {
    const long long nvec = a.n >> 3;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec;
         i += (long long)gridDim.x * blockDim.x) {
      float g[8];
      if (USE_MC) {
        const __nv_bfloat16* src = reinterpret_cast<const __nv_bfloat16*>(a.mc_grads) + a.shard_lo + i * 8;
        uint32_t r0, r1, r2, r3;
        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                     : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                     : "l"(src)
                     : "memory");
        float2 f0 = unpack_bf16x2(r0), f1 = unpack_bf16x2(r1), f2 = unpack_bf16x2(r2), f3 = unpack_bf16x2(r3);
        g[0] = f0.x; g[1] = f0.y; g[2] = f1.x; g[3] = f1.y; g[4] = f2.x; g[5] = f2.y; g[6] = f3.x; g[7] = f3.y;
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) g[j] = 0.f;
        // two batches of four peers: four 16-byte loads in flight, then accumulate
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint4 u[4];
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const int r = half * 4 + q;
            if (r < a.world) {
              // start with the next rank after mine so the ranks do not all hit the same peer at once
              int src_rank = a.my_rank + 1 + r;
              if (src_rank >= a.world) src_rank -= a.world;
              const __nv_bfloat16* src =
                  reinterpret_cast<const __nv_bfloat16*>(a.grads.p[src_rank]) + a.shard_lo + i * 8;
              u[q] = *reinterpret_cast<const uint4*>(src);
            }
          }
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            if (half * 4 + q < a.world) {
              float2 f0 = unpack_bf16x2(u[q].x), f1 = unpack_bf16x2(u[q].y), f2 = unpack_bf16x2(u[q].z),
                     f3 = unpack_bf16x2(u[q].w);
              g[0] += f0.x; g[1] += f0.y; g[2] += f1.x; g[3] += f1.y;
              g[4] += f2.x; g[5] += f2.y; g[6] += f3.x; g[7] += f3.y;
            }
          }
        }
      }
      if (REDUCE_ONLY) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          g[j] *= a.grad_scale;
          sq += g[j] * g[j];
        }
        reinterpret_cast<float4*>(a.grad_out)[i * 2] = *reinterpret_cast<float4*>(g);
        reinterpret_cast<float4*>(a.grad_out)[i * 2 + 1] = *reinterpret_cast<float4*>(g + 4);
        continue;
      }
      float pv[8], mv[8], vv[8];
      *reinterpret_cast<float4*>(pv) = reinterpret_cast<const float4*>(a.master)[i * 2];
      *reinterpret_cast<float4*>(pv + 4) = reinterpret_cast<const float4*>(a.master)[i * 2 + 1];
      *reinterpret_cast<float4*>(mv) = reinterpret_cast<const float4*>(a.m)[i * 2];
      *reinterpret_cast<float4*>(mv + 4) = reinterpret_cast<const float4*>(a.m)[i * 2 + 1];
      *reinterpret_cast<float4*>(vv) = reinterpret_cast<const float4*>(a.v)[i * 2];
      *reinterpret_cast<float4*>(vv + 4) = reinterpret_cast<const float4*>(a.v)[i * 2 + 1];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float gj = g[j] * a.grad_scale;
        mv[j] = a.beta1 * mv[j] + (1.f - a.beta1) * gj;
        vv[j] = a.beta2 * vv[j] + (1.f - a.beta2) * gj * gj;
        const float mh = mv[j] / bc1, vh = vv[j] / bc2;
        pv[j] = pv[j] * (1.f - a.lr * a.wd) - a.lr * mh / (sqrtf(vh) + a.eps);
      }
      reinterpret_cast<float4*>(a.master)[i * 2] = *reinterpret_cast<float4*>(pv);
      reinterpret_cast<float4*>(a.master)[i * 2 + 1] = *reinterpret_cast<float4*>(pv + 4);
      reinterpret_cast<float4*>(a.m)[i * 2] = *reinterpret_cast<float4*>(mv);
      reinterpret_cast<float4*>(a.m)[i * 2 + 1] = *reinterpret_cast<float4*>(mv + 4);
      reinterpret_cast<float4*>(a.v)[i * 2] = *reinterpret_cast<float4*>(vv);
      reinterpret_cast<float4*>(a.v)[i * 2 + 1] = *reinterpret_cast<float4*>(vv + 4);
      if (a.p_lp) {
        uint4 o;
        o.x = pack_bf16x2(pv[0], pv[1]); o.y = pack_bf16x2(pv[2], pv[3]);
        o.z = pack_bf16x2(pv[4], pv[5]); o.w = pack_bf16x2(pv[6], pv[7]);
        reinterpret_cast<uint4*>(a.p_lp)[i] = o;
      }
    }
  }
  if (REDUCE_ONLY) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, off);
    if ((threadIdx.x & 31) == 0) s_sq[threadIdx.x >> 5] = sq;
    __syncthreads();
    if (threadIdx.x == 0) {
      float t = 0.f;
      for (int w = 0; w < 8; ++w) t += s_sq[w];
      atomicAdd(a.sumsq, t);
    }
  }
  // last block to finish tells every rank that their gradient buffer has been consumed by this rank and
  // that this rank's weight shard now holds the new version
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int prev = atomicAdd(a.done_counter, 1);
    s_ok = (prev == (int)gridDim.x - 1) ? 1 : 0;
  }
  __syncthreads();
  if (s_ok && threadIdx.x < a.world) {
    __threadfence_system();
    st_release_sys(a.pads.p[threadIdx.x] + a.consumed_idx + a.my_rank, a.consumed_val + ep);
    if (a.version_idx >= 0) st_release_sys(a.pads.p[threadIdx.x] + a.version_idx + a.my_rank, a.version_val + ep);
    if (threadIdx.x == 0) *a.done_counter = 0;
  }
}

// ------------------------------------------------------------------ all-gather (pull)
struct AgArgs {
  PeerPtrs shards;          // every rank's bf16 shard (symmetric)
  __nv_bfloat16* full;      // local gathered buffer [world * shard_elems]
  long long shard_elems;    // multiple of 8
  int world, my_rank;
  const int* local_pad;
  int version_idx;          // wait: local_pad[version_idx + r] >= version_val before copying rank r's shard
  int version_val;
  int* ready_flags;         // local int[world]: set to ready_val once shard r has landed (gpu scope)
  int ready_val;
  int* block_counters;      // local int[world], zero before launch; reset when a shard completes
  int blocks_per_shard;
  uint32_t wait_limit;
  int* status;
  const int* epoch;         // optional device counter added to version_val (graph replays)
};

// grid = world * blocks_per_shard; block b copies a slice of shard (my_rank + 1 + b / blocks_per_shard) % world,
// so the local shard (cheap) comes last and remote traffic starts at once, staggered across ranks.
__global__ void __launch_bounds__(256, 4)
allgather_pull_kernel(const AgArgs a) {
  __shared__ int s_ok;
  const int order = blockIdx.x / a.blocks_per_shard;
  const int slice = blockIdx.x % a.blocks_per_shard;
  int src = a.my_rank + 1 + order;
  if (src >= a.world) src -= a.world;
  if (threadIdx.x == 0) {
    bool ok = true;
    if (src != a.my_rank)
      ok = wait_flag_ge(a.local_pad + a.version_idx + src, a.version_val + (a.epoch ? *a.epoch : 0), a.wait_limit);
    s_ok = ok ? 1 : 0;
    if (!ok && a.status) atomicCAS(a.status, 0, GF_ERR_WAIT_PEER);
  }
  __syncthreads();
  if (s_ok) {
    const long long nvec = a.shard_elems >> 3;
    const long long per = (nvec + a.blocks_per_shard - 1) / a.blocks_per_shard;
    const long long lo = slice * per;
    long long hi = lo + per;
    if (hi > nvec) hi = nvec;
    const uint4* s = reinterpret_cast<const uint4*>(a.shards.p[src]);
    uint4* d = reinterpret_cast<uint4*>(a.full + (long long)src * a.shard_elems);
    long long i = lo + threadIdx.x;
    // eight independent 16-byte loads in flight per thread (NVLink latency is a few microseconds, so the
    // kernel needs megabytes in flight to fill the links)
    const long long bd = blockDim.x;
    for (; i + 7 * bd < hi; i += 8 * bd) {
      uint4 v[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) v[k] = s[i + k * bd];
#pragma unroll
      for (int k = 0; k < 8; ++k) d[i + k * bd] = v[k];
    }
    for (; i < hi; i += blockDim.x) d[i] = s[i];
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int prev = atomicAdd(a.block_counters + src, 1);
    if (prev == a.blocks_per_shard - 1) {
      a.block_counters[src] = 0;
      __threadfence();
      if (s_ok) st_release_gpu(a.ready_flags + src, a.ready_val);
    }
  }
}

__global__ void counter_add_kernel(int* p, int delta) { *p += delta; }

__global__ void fill_int_kernel(int* p, int n, int v) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) p[i] = v;
}

}  // namespace gf

using namespace gf;

static void configure_comm_kernels() {
  static gf::DeviceOnce done;
  if (!done.todo()) return;
  prefer_max_smem(signal_peers_kernel);
  prefer_max_smem(wait_flags_kernel);
  prefer_max_smem(rs_adamw_kernel<true>);
  prefer_max_smem(rs_adamw_kernel<false>);
  prefer_max_smem(rs_adamw_kernel<true, true>);
  prefer_max_smem(rs_adamw_kernel<false, true>);
  prefer_max_smem(allgather_pull_kernel);
  prefer_max_smem(fill_int_kernel);
  prefer_max_smem(counter_add_kernel);
  done.mark();
}

static inline uint32_t limit_or_default(long long wait_limit) {
  return wait_limit > 0 ? (uint32_t)wait_limit : (uint32_t)(1u << 24);  // x 100 ns sleeps: about 2 s
}

// pads: device pointers (as uint64) of every rank's signal pad, world entries.
// The *_ep variants take `epoch`, a device int (or null) whose current value is added to every flag value of the
// launch. A training step recorded once in a CUDA graph bumps that counter with gf_counter_add at its start, so
// every replay publishes and expects new flag values although the launch arguments are frozen.
GF_API int gf_signal_peers_ep(const unsigned long long* pads, int world, int my_rank, int idx_base, int value,
                              const int* epoch, void* stream) {
  gf::enter();
  configure_comm_kernels();
  if (world < 1 || world > MAX_RANKS) return GFH_BAD_ARG;
  PeerFlagPtrs pp;
  for (int r = 0; r < MAX_RANKS; ++r) pp.p[r] = r < world ? reinterpret_cast<int*>(pads[r]) : nullptr;
  signal_peers_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(pp, idx_base, my_rank, world, value, epoch);
  return cudaGetLastError() == cudaSuccess ? GFH_OK : GFH_CUDA;
}

GF_API int gf_signal_peers(const unsigned long long* pads, int world, int my_rank, int idx_base, int value,
                           void* stream) {
  return gf_signal_peers_ep(pads, world, my_rank, idx_base, value, nullptr, stream);
}

GF_API int gf_counter_add(int* counter, int delta, void* stream) {
  gf::enter();
  configure_comm_kernels();
  if (!counter) return GFH_BAD_ARG;
  counter_add_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(counter, delta);
  return cudaGetLastError() == cudaSuccess ? GFH_OK : GFH_CUDA;
}

GF_API int gf_wait_flags_ep(const int* local_pad, int idx_base, int world, int value, long long wait_limit,
                            int* status, const int* epoch, void* stream) {
  gf::enter();
  configure_comm_kernels();
  if (world < 1 || world > 32) return GFH_BAD_ARG;
  wait_flags_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(local_pad, idx_base, world, value,
                                                        limit_or_default(wait_limit), status, epoch);
  return cudaGetLastError() == cudaSuccess ? GFH_OK : GFH_CUDA;
}

GF_API int gf_wait_flags(const int* local_pad, int idx_base, int world, int value, long long wait_limit, int* status,
                         void* stream) {
  return gf_wait_flags_ep(local_pad, idx_base, world, value, wait_limit, status, nullptr, stream);
}

GF_API int gf_fill_int(int* p, int n, int v, void* stream) {
  gf::enter();
  configure_comm_kernels();
  fill_int_kernel<<<(n + 255) / 256, 256, 0, (cudaStream_t)stream>>>(p, n, v);
  return cudaGetLastError() == cudaSuccess ? GFH_OK : GFH_CUDA;
}

// grad_ptrs / pads: world device pointers each. mc_grads: multicast pointer of the gradient buffer or 0.
// With `epoch` the Adam step number is *epoch (bias corrections computed on the device) and `step` is ignored.
GF_API int gf_rs_adamw_fused_ep(const unsigned long long* grad_ptrs, unsigned long long mc_grads,
                                const unsigned long long* pads, int world, int my_rank, long long shard_lo, long long n,
                                float* master, float* m, float* v, void* p_lp, float lr, float beta1, float beta2,
                                float eps, float wd, int step, float grad_scale, int ready_idx, int ready_val,
                                int consumed_idx, int consumed_val, int version_idx, int version_val,
                                int* done_counter, int max_ctas, long long wait_limit, int* status, const int* epoch,
                                void* stream) {
  gf::enter();
  configure_comm_kernels();
  if (world < 1 || world > MAX_RANKS || (n & 7) || (shard_lo & 7)) return GFH_BAD_ARG;
  RsAdamArgs a;
  for (int r = 0; r < MAX_RANKS; ++r) {
    a.grads.p[r] = r < world ? reinterpret_cast<const void*>(grad_ptrs[r]) : nullptr;
    a.pads.p[r] = r < world ? reinterpret_cast<int*>(pads[r]) : nullptr;
  }
  a.mc_grads = reinterpret_cast<const void*>(mc_grads);
  a.shard_lo = shard_lo; a.n = n; a.master = master; a.m = m; a.v = v; a.p_lp = (__nv_bfloat16*)p_lp;
  a.lr = lr; a.beta1 = beta1; a.beta2 = beta2; a.eps = eps; a.wd = wd; a.grad_scale = grad_scale;
  a.bc1 = 1.f - powf(beta1, (float)step);
  a.bc2 = 1.f - powf(beta2, (float)step);
  a.world = world; a.my_rank = my_rank;
  a.local_pad = a.pads.p[my_rank];
  a.ready_idx = ready_idx; a.ready_val = ready_val; a.consumed_idx = consumed_idx; a.consumed_val = consumed_val;
  a.version_idx = version_idx; a.version_val = version_val;
  a.done_counter = done_counter; a.wait_limit = limit_or_default(wait_limit); a.status = status;
  a.grad_out = nullptr; a.sumsq = nullptr;
  a.epoch = epoch; a.step_from_epoch = epoch ? 1 : 0;
  long long want = ((n >> 3) + 255) / 256;
  int grid = max_ctas > 0 ? max_ctas : sm_count();
  if (want < grid) grid = (int)(want > 0 ? want : 1);
  if (mc_grads)
    rs_adamw_kernel<true><<<grid, 256, 0, (cudaStream_t)stream>>>(a);
  else
    rs_adamw_kernel<false><<<grid, 256, 0, (cudaStream_t)stream>>>(a);
  return cudaGetLastError() == cudaSuccess ? GFH_OK : GFH_CUDA;
}

GF_API int gf_rs_adamw_fused(const unsigned long long* grad_ptrs, unsigned long long mc_grads,
                             const unsigned long long* pads, int world, int my_rank, long long shard_lo, long long n,
                             float* master, float* m, float* v, void* p_lp, float lr, float beta1, float beta2,
                             float eps, float wd, int step, float grad_scale, int ready_idx, int ready_val,
                             int consumed_idx, int consumed_val, int version_idx, int version_val, int* done_counter,
                             int max_ctas, long long wait_limit, int* status, void* stream) {
  return gf_rs_adamw_fused_ep(grad_ptrs, mc_grads, pads, world, my_rank, shard_lo, n, master, m, v, p_lp, lr, beta1,
                              beta2, eps, wd, step, grad_scale, ready_idx, ready_val, consumed_idx, consumed_val,
                              version_idx, version_val, done_counter, max_ctas, wait_limit, status, nullptr, stream);
}

// Reduce-scatter alone, for steps that need the global gradient norm before they may update (clipping, overflow
// check): this rank's slice of every rank's gradient buffer is summed in fp32, multiplied by grad_scale and written
// to grad_out (fp32 [n]); the sum of its squares is ADDED to *sumsq (zero it once per step). Flags as in
// gf_rs_adamw_fused, except that no weight version is published.
GF_API int gf_rs_reduce_only(const unsigned long long* grad_ptrs, unsigned long long mc_grads,
                             const unsigned long long* pads, int world, int my_rank, long long shard_lo, long long n,
                             float* grad_out, float* sumsq, float grad_scale, int ready_idx, int ready_val,
                             int consumed_idx, int consumed_val, int* done_counter, int max_ctas, long long wait_limit,
                             int* status, void* stream) {
  gf::enter();
  configure_comm_kernels();
  if (world < 1 || world > MAX_RANKS || (n & 7) || (shard_lo & 7) || !grad_out || !sumsq) return GFH_BAD_ARG;
  RsAdamArgs a;
  for (int r = 0; r < MAX_RANKS; ++r) {
    a.grads.p[r] = r < world ? reinterpret_cast<const void*>(grad_ptrs[r]) : nullptr;
    a.pads.p[r] = r < world ? reinterpret_cast<int*>(pads[r]) : nullptr;
  }
  a.mc_grads = reinterpret_cast<const void*>(mc_grads);
  a.shard_lo = shard_lo; a.n = n; a.master = nullptr; a.m = nullptr; a.v = nullptr; a.p_lp = nullptr;
  a.lr = 0.f; a.beta1 = 0.f; a.beta2 = 0.f; a.eps = 0.f; a.wd = 0.f; a.grad_scale = grad_scale; a.bc1 = 1.f; a.bc2 = 1.f;
  a.world = world; a.my_rank = my_rank;
  a.local_pad = a.pads.p[my_rank];
  a.ready_idx = ready_idx; a.ready_val = ready_val; a.consumed_idx = consumed_idx; a.consumed_val = consumed_val;
  a.version_idx = -1; a.version_val = 0;
  a.done_counter = done_counter; a.wait_limit = limit_or_default(wait_limit); a.status = status;
  a.grad_out = grad_out; a.sumsq = sumsq;
  a.epoch = nullptr; a.step_from_epoch = 0;
  long long want = ((n >> 3) + 255) / 256;
  int grid = max_ctas > 0 ? max_ctas : sm_count();
  if (want < grid) grid = (int)(want > 0 ? want : 1);
  if (mc_grads)
    rs_adamw_kernel<true, true><<<grid, 256, 0, (cudaStream_t)stream>>>(a);
  else
    rs_adamw_kernel<false, true><<<grid, 256, 0, (cudaStream_t)stream>>>(a);
  return cudaGetLastError() == cudaSuccess ? GFH_OK : GFH_CUDA;
}

// shard_ptrs: every rank's shard (world pointers). ready_flags / block_counters: local int[world].
GF_API int gf_allgather_pull_ep(const unsigned long long* shard_ptrs, void* full, long long shard_elems, int world,
                                int my_rank, const int* local_pad, int version_idx, int version_val,
                                int* ready_flags, int ready_val, int* block_counters, int blocks_per_shard,
                                long long wait_limit, int* status, const int* epoch, void* stream) {
  gf::enter();
  configure_comm_kernels();
  if (world < 1 || world > MAX_RANKS || (shard_elems & 7) || blocks_per_shard < 1) return GFH_BAD_ARG;
  AgArgs a;
  for (int r = 0; r < MAX_RANKS; ++r) a.shards.p[r] = r < world ? reinterpret_cast<const void*>(shard_ptrs[r]) : nullptr;
  a.full = (__nv_bfloat16*)full; a.shard_elems = shard_elems; a.world = world; a.my_rank = my_rank;
  a.local_pad = local_pad; a.version_idx = version_idx; a.version_val = version_val;
  a.ready_flags = ready_flags; a.ready_val = ready_val; a.block_counters = block_counters;
  a.blocks_per_shard = blocks_per_shard; a.wait_limit = limit_or_default(wait_limit); a.status = status;
  a.epoch = epoch;
  allgather_pull_kernel<<<world * blocks_per_shard, 256, 0, (cudaStream_t)stream>>>(a);
  return cudaGetLastError() == cudaSuccess ? GFH_OK : GFH_CUDA;
}

GF_API int gf_allgather_pull(const unsigned long long* shard_ptrs, void* full, long long shard_elems, int world,
                             int my_rank, const int* local_pad, int version_idx, int version_val, int* ready_flags,
                             int ready_val, int* block_counters, int blocks_per_shard, long long wait_limit,
                             int* status, void* stream) {
  return gf_allgather_pull_ep(shard_ptrs, full, shard_elems, world, my_rank, local_pad, version_idx, version_val,
                              ready_flags, ready_val, block_counters, blocks_per_shard, wait_limit, status, nullptr,
                              stream);
}

// ------------------------------------------------------------------------------------------------------------
// One-shot all-reduce fused with the residual add and RMSNorm that follow a row-parallel projection in a
// tensor-parallel decode step. Every rank holds a partial product [rows, d] (bf16) in peer-mapped memory; the
// kernel of every rank reads all partials, adds the residual stream, writes the new residual h and its normalised
// copy x (both replicated), so the next column-parallel projection needs no all-gather. One launch replaces
// reduce-scatter + add + RMSNorm + all-gather.
//
// Synchronisation is entirely on the device, which makes the kernel replayable from a CUDA graph: the call number
// is a device counter (`epoch`, bumped by the last CTA), a rank publishes "my partial of call e is written" with a
// release store of e into every peer's flag array, and waits (bounded) until all peers' flags reach e. Partials are
// double-buffered by call parity (given by the host; a rank can be at most one call ahead of a peer).
namespace gf {
struct ArPeers {
  const __nv_bfloat16* partial[8];   // every rank's partial buffer of the current parity
  int* flags[8];                     // every rank's flag array int[8], indexed by source rank
};

__global__ void __launch_bounds__(256)
allreduce_residual_rmsnorm_kernel(ArPeers peers, int world, int rank, int* __restrict__ epoch_counter,
                                  int* __restrict__ done_counter, const __nv_bfloat16* __restrict__ residual,
                                  const __nv_bfloat16* __restrict__ norm_w, float eps, __nv_bfloat16* __restrict__ h_out,
                                  __nv_bfloat16* __restrict__ x_out, int rows, int d, long long wait_limit,
                                  int* status) {
  __shared__ int s_ok;
  __shared__ float red[32];
  const int epoch = *reinterpret_cast<volatile int*>(epoch_counter) + 1;
  if (threadIdx.x == 0) {
    if (blockIdx.x == 0) {
      __threadfence_system();          // the partial written by the preceding kernels of this stream
      for (int r = 0; r < world; ++r)
        asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(peers.flags[r] + rank), "r"(epoch) : "memory");
    }
    int ok = 1;
    for (int r = 0; r < world && ok; ++r) {
      long long it = 0;
      while (true) {
        int v;
        asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(peers.flags[rank] + r) : "memory");
        if (v >= epoch) break;
        if (++it > wait_limit) { ok = 0; break; }
        __nanosleep(32);
      }
    }
    if (!ok && status) atomicCAS(status, 0, GF_ERR_WAIT_PEER);
    s_ok = ok;
  }
  __syncthreads();
  if (s_ok) {
    const int nv = d >> 3;
    for (int row = blockIdx.x; row < rows; row += gridDim.x) {
      float sq = 0.f;
      // pass 1: sum of partials + residual -> h (kept in registers for up to 4 vectors per thread). The peer loads
      // of two vectors (up to 16 loads of 16 bytes) are issued before any of them is used: a peer load costs a
      // few microseconds of NVLink latency, so they must overlap.
      float hv[4][8];
#pragma unroll
      for (int i0 = 0; i0 < 4; i0 += 2) {
        uint4 pu[2][8];
        uint4 ru[2];
#pragma unroll
        for (int k = 0; k < 2; ++k) {
          const int v = threadIdx.x + (i0 + k) * 256;
          if (v < nv) {
            ru[k] = *reinterpret_cast<const uint4*>(residual + (long long)row * d + v * 8);
#pragma unroll
            for (int r = 0; r < 8; ++r)
              pu[k][r] = r < world ? *reinterpret_cast<const uint4*>(peers.partial[r] + (long long)row * d + v * 8)
                                   : make_uint4(0, 0, 0, 0);
          }
        }
#pragma unroll
        for (int k = 0; k < 2; ++k) {
          const int i = i0 + k;
          const int v = threadIdx.x + i * 256;
          if (v < nv) {
            float acc[8];
            {
              float2 a = unpack_bf16x2(ru[k].x), b = unpack_bf16x2(ru[k].y), c = unpack_bf16x2(ru[k].z), e = unpack_bf16x2(ru[k].w);
              acc[0] = a.x; acc[1] = a.y; acc[2] = b.x; acc[3] = b.y; acc[4] = c.x; acc[5] = c.y; acc[6] = e.x; acc[7] = e.y;
            }
#pragma unroll
            for (int r = 0; r < 8; ++r) {
              const uint4 u = pu[k][r];
              float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), e = unpack_bf16x2(u.w);
              acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y;
              acc[4] += c.x; acc[5] += c.y; acc[6] += e.x; acc[7] += e.y;
            }
            uint4 o;
            o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);
            o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
            *reinterpret_cast<uint4*>(h_out + (long long)row * d + v * 8) = o;
            // the normalisation uses the bf16-rounded h, like a separate RMSNorm kernel reading h would
            float2 a = unpack_bf16x2(o.x), b = unpack_bf16x2(o.y), c = unpack_bf16x2(o.z), e = unpack_bf16x2(o.w);
            hv[i][0] = a.x; hv[i][1] = a.y; hv[i][2] = b.x; hv[i][3] = b.y;
            hv[i][4] = c.x; hv[i][5] = c.y; hv[i][6] = e.x; hv[i][7] = e.y;
#pragma unroll
            for (int j = 0; j < 8; ++j) sq += hv[i][j] * hv[i][j];
          }
        }
      }
      for (int o = 16; o; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
      if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = sq;
      __syncthreads();
      float tot = 0.f;
      for (int w = 0; w < 8; ++w) tot += red[w];
      __syncthreads();
      const float rstd = rsqrtf(tot / (float)d + eps);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int v = threadIdx.x + i * 256;
        if (v < nv) {
          const uint4 wu = *reinterpret_cast<const uint4*>(norm_w + v * 8);
          float2 a = unpack_bf16x2(wu.x), b = unpack_bf16x2(wu.y), c = unpack_bf16x2(wu.z), e = unpack_bf16x2(wu.w);
          uint4 o;
          o.x = pack_bf16x2(hv[i][0] * rstd * a.x, hv[i][1] * rstd * a.y);
          o.y = pack_bf16x2(hv[i][2] * rstd * b.x, hv[i][3] * rstd * b.y);
          o.z = pack_bf16x2(hv[i][4] * rstd * c.x, hv[i][5] * rstd * c.y);
          o.w = pack_bf16x2(hv[i][6] * rstd * e.x, hv[i][7] * rstd * e.y);
          *reinterpret_cast<uint4*>(x_out + (long long)row * d + v * 8) = o;
        }
      }
    }
  }
  // the last CTA advances the call counter (all CTAs have read it by now: they are past the first barrier)
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const int done = atomicAdd(done_counter, 1);
    if (done == (int)gridDim.x - 1) {
      *done_counter = 0;
      *epoch_counter = epoch;
      __threadfence();
    }
  }
}
}  // namespace gf

// partial_ptrs / flag_ptrs: `world` device addresses (peer-mapped). rows x d bf16, d % 8 == 0 and d <= 8192.
GF_API int gf_allreduce_residual_rmsnorm(const unsigned long long* partial_ptrs, const unsigned long long* flag_ptrs,
                                         int world, int rank, int* epoch_counter, int* done_counter,
                                         const void* residual, const void* norm_w, float eps, void* h_out, void* x_out,
                                         int rows, int d, long long wait_limit, int* status, void* stream) {
  gf::enter();
  if (world < 1 || world > 8 || rows <= 0 || (d & 7) || d > 8192) return GFH_BAD_ARG;
  gf::ArPeers peers;
  for (int i = 0; i < 8; ++i) {
    peers.partial[i] = i < world ? reinterpret_cast<const __nv_bfloat16*>(partial_ptrs[i]) : nullptr;
    peers.flags[i] = i < world ? reinterpret_cast<int*>(flag_ptrs[i]) : nullptr;
  }
  int grid = rows < 148 ? rows : 148;
  gf::allreduce_residual_rmsnorm_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(
      peers, world, rank, epoch_counter, done_counter, (const __nv_bfloat16*)residual, (const __nv_bfloat16*)norm_w, eps,
      (__nv_bfloat16*)h_out, (__nv_bfloat16*)x_out, rows, d, limit_or_default(wait_limit), status);
  return cudaGetLastError() == cudaSuccess ? GFH_OK : GFH_CUDA;
}
