// Collectives over NVLink peer memory for one process per GPU.
//
// Every rank maps the same symmetric buffer of all peers (the Python side exchanges the
// mappings), so a kernel can read or write any rank's shard with plain loads and stores.
// Ordering between ranks uses 32-bit epoch flags inside the symmetric buffer:
//   flag[slot][src_rank] on rank r  =  "src_rank has reached epoch e for this slot"
// A producer publishes with a system-scope release after its data is written; a consumer
// spins with system-scope acquires, for a bounded number of polls, and records
// FSB_ERR_WAIT_TIMEOUT_PEER in the status word when the flag never arrives (the kernel then
// skips its work and returns, so the context stays usable).
//
// Kernels:
//   signal        publish an epoch to every peer's flag row
//   gather_pull   wait for the peers' epoch, then copy a list of (peer source -> local
//                 destination) segments: all-gather and copy-out into per-parameter buffers
//                 in one pass (replaces NCCL all-gather + the strided copy-out)
//   reduce_adamw  wait for the peers' epoch, then for every element of this rank's shard sum
//                 the W peers' gradient rows in rank order (deterministic), scale, apply AdamW
//                 to the bf16/fp32 master shard and fp32 moments: reduce-scatter, cast/scale
//                 and the sharded optimizer in one pass over the data
//   reduce_pull   the same reduction without the optimizer
#include "common.cuh"

namespace {
using namespace fsb;

constexpr int MAX_RANKS = 16;
constexpr int kMaxLocalExperts = 256;

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Returns false on timeout, or as soon as the status word shows that some wait of this process has already
// failed (after the first failure the step's result is lost anyway; without this every later wait would sit
// out its own limit and a protocol error would look like a hang). Epochs only grow, so ">= epoch" also
// accepts a peer that is ahead.
__device__ __forceinline__ bool wait_flag(const uint32_t* p, uint32_t epoch, uint32_t max_polls,
                                          const volatile int* status) {
  for (uint32_t i = 0; i < max_polls; ++i) {
    if (static_cast<int32_t>(ld_acquire_sys(p) - epoch) >= 0) return true;
    if (i > 64) __nanosleep(200);
    if ((i & 1023) == 1023 && *status != 0) return false;
  }
  return false;
}

// The status record: [0] error code, then (written by the first failed wait only) [1],[2] the address of the
// flag that never arrived, [3] the epoch waited for, [4] the peer's rank in the group, [5] the value last seen.
constexpr int kStatusInts = 8;
__device__ __forceinline__ void report_wait_failure(int* status, const uint32_t* flag, uint32_t epoch, int peer) {
  if (atomicCAS(status, 0, FSB_ERR_WAIT_TIMEOUT_PEER) == 0) {
    const unsigned long long a = reinterpret_cast<unsigned long long>(flag);
    status[1] = static_cast<int>(a & 0xffffffffu);
    status[2] = static_cast<int>(a >> 32);
    status[3] = static_cast<int>(epoch);
    status[4] = peer;
    status[5] = static_cast<int>(ld_acquire_sys(flag));
    __threadfence_system();
  }
}

// All threads of the CTA return the same verdict.
__device__ __forceinline__ bool cta_wait_peers(const uint32_t* my_flags, int world, uint32_t epoch,
                                               uint32_t max_polls, int* status) {
  __shared__ int s_ok;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (threadIdx.x < world) {
    if (!wait_flag(my_flags + threadIdx.x, epoch, max_polls, status)) {
      s_ok = 0;
      report_wait_failure(status, my_flags + threadIdx.x, epoch, threadIdx.x);
    }
  }
  __syncthreads();
  return s_ok != 0;
}

struct PeerPtrs {
  void* p[MAX_RANKS];
};

// Sum of the same 16 bytes of every rank's copy of a multicast-bound symmetric buffer, added inside
// the NVSwitch: one load crosses this GPU's links instead of one per peer. `mc` is an address in
// the multicast mapping. The switch's summation order is fixed for a given set of ranks.
__device__ __forceinline__ float4 multimem_sum_f32x4(const void* mc) {
  float4 r;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(r.x), "=f"(r.y), "=f"(r.z), "=f"(r.w)
               : "l"(mc)
               : "memory");
  return r;
}

__global__ void signal_kernel(PeerPtrs flags, int rank, int world, uint32_t epoch) {
  // flags.p[r] = address of this slot's flag row on rank r
  if (threadIdx.x < world) {
    __threadfence_system();
    st_release_sys(static_cast<uint32_t*>(flags.p[threadIdx.x]) + rank, epoch);
  }
}

__global__ void wait_kernel(const uint32_t* my_flags, int world, uint32_t epoch, uint32_t max_polls,
                            int* status) {
  cta_wait_peers(my_flags, world, epoch, max_polls, status);
}

struct SegDesc {
  const void* src;
  void* dst;
  long long n;  // bytes
  int mode;
  int pad;
};

__global__ void gather_pull_kernel(const SegDesc* __restrict__ descs, const uint32_t* my_flags, int world,
                                   uint32_t epoch, uint32_t max_polls, int* status) {
  if (my_flags != nullptr && !cta_wait_peers(my_flags, world, epoch, max_polls, status)) return;
  const SegDesc d = descs[blockIdx.y];
  const long long tid = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const uintptr_t al = reinterpret_cast<uintptr_t>(d.src) | reinterpret_cast<uintptr_t>(d.dst);
  if ((al & 15) == 0) {
    const long long nv = d.n / 16;
    const uint4* s = static_cast<const uint4*>(d.src);
    uint4* t = static_cast<uint4*>(d.dst);
    // four independent 16-byte loads in flight per thread: NVLink latency is long
    long long i = tid;
    for (; i + 3 * stride < nv; i += 4 * stride) {
      const uint4 a = s[i], b = s[i + stride], c = s[i + 2 * stride], e = s[i + 3 * stride];
      t[i] = a; t[i + stride] = b; t[i + 2 * stride] = c; t[i + 3 * stride] = e;
    }
    for (; i < nv; i += stride) t[i] = s[i];
    for (long long j = nv * 16 + tid; j < d.n; j += stride)
      static_cast<uint8_t*>(d.dst)[j] = static_cast<const uint8_t*>(d.src)[j];
  } else {
    for (long long j = tid; j < d.n; j += stride)
      static_cast<uint8_t*>(d.dst)[j] = static_cast<const uint8_t*>(d.src)[j];
  }
}

struct AdamArgs {
  float lr, beta1, beta2, eps, weight_decay, bias1, bias2_sqrt;
};

// rows.p[r] = address of rank r's gradient row that belongs to THIS rank (fp32, n elements).
// With MC, rows.p[0] is instead the address of that row in the multicast mapping of the symmetric
// buffer (the row sits at the same offset on every rank) and the W-way sum happens in the switch.
template <typename PT, bool WITH_ADAM, bool MC>
__global__ void __launch_bounds__(256)
reduce_rows_kernel(PeerPtrs rows, int world, long long n, float scale, float* __restrict__ g_out,
                   PT* __restrict__ p, float* __restrict__ m, float* __restrict__ v, AdamArgs a,
                   const uint32_t* my_flags, uint32_t epoch, uint32_t max_polls, int* status) {
  if (my_flags != nullptr && !cta_wait_peers(my_flags, world, epoch, max_polls, status)) return;
  if (MC) __threadfence_system();
  const long long tid = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long n4 = n / 4;
  for (long long i = tid; i < n4; i += stride) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    if (MC) {
      acc = multimem_sum_f32x4(static_cast<const float4*>(rows.p[0]) + i);
    } else {
      for (int r = 0; r < world; ++r) {  // fixed rank order: the sum is deterministic
        const float4 t = static_cast<const float4*>(rows.p[r])[i];
        acc.x += t.x; acc.y += t.y; acc.z += t.z; acc.w += t.w;
      }
    }
    float g[4] = {acc.x * scale, acc.y * scale, acc.z * scale, acc.w * scale};
    if (g_out) *reinterpret_cast<float4*>(g_out + i * 4) = make_float4(g[0], g[1], g[2], g[3]);
    if (WITH_ADAM) {
      const float4 mv = *reinterpret_cast<const float4*>(m + i * 4);
      const float4 vv = *reinterpret_cast<const float4*>(v + i * 4);
      float mm[4] = {mv.x, mv.y, mv.z, mv.w}, vq[4] = {vv.x, vv.y, vv.z, vv.w};
      float pv[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) pv[j] = static_cast<float>(p[i * 4 + j]);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        pv[j] *= (1.f - a.lr * a.weight_decay);
        mm[j] = mm[j] + (1.f - a.beta1) * (g[j] - mm[j]);
        vq[j] = a.beta2 * vq[j] + (1.f - a.beta2) * g[j] * g[j];
        pv[j] -= (a.lr / a.bias1) * (mm[j] / (sqrtf(vq[j]) / a.bias2_sqrt + a.eps));
        p[i * 4 + j] = static_cast<PT>(pv[j]);
      }
      *reinterpret_cast<float4*>(m + i * 4) = make_float4(mm[0], mm[1], mm[2], mm[3]);
      *reinterpret_cast<float4*>(v + i * 4) = make_float4(vq[0], vq[1], vq[2], vq[3]);
    }
  }
  if (MC) return;   // the launcher only takes the multicast path for n % 4 == 0
  for (long long i = n4 * 4 + tid; i < n; i += stride) {
    float acc = 0.f;
    for (int r = 0; r < world; ++r) acc += static_cast<const float*>(rows.p[r])[i];
    const float g = acc * scale;
    if (g_out) g_out[i] = g;
    if (WITH_ADAM) {
      float pv = static_cast<float>(p[i]) * (1.f - a.lr * a.weight_decay);
      const float mm = m[i] + (1.f - a.beta1) * (g - m[i]);
      const float vq = a.beta2 * v[i] + (1.f - a.beta2) * g * g;
      pv -= (a.lr / a.bias1) * (mm / (sqrtf(vq) / a.bias2_sqrt + a.eps));
      p[i] = static_cast<PT>(pv);
      m[i] = mm;
      v[i] = vq;
    }
  }
}

inline int grid_for(long long n, int per_thread) {
  long long b = (n + 256LL * per_thread - 1) / (256LL * per_thread);
  if (b < 1) b = 1;
  if (b > 148 * 8) b = 148 * 8;
  return static_cast<int>(b);
}
inline int ok() { return cudaGetLastError() == cudaSuccess ? FSB_OK : FSB_ERR_LAUNCH; }

}  // namespace

// flag_rows[r]: address (in this process's address space) of the slot's flag row on rank r.
FSB_API int fsb_comm_signal(const unsigned long long* flag_rows, int rank, int world, unsigned epoch,
                            cudaStream_t stream) {
  if (world > MAX_RANKS) return FSB_ERR_TOO_LARGE;
  PeerPtrs f;
  for (int r = 0; r < world; ++r) f.p[r] = reinterpret_cast<void*>(flag_rows[r]);
  signal_kernel<<<1, 32, 0, stream>>>(f, rank, world, epoch);
  return ok();
}

FSB_API int fsb_comm_wait(const void* my_flags, int world, unsigned epoch, unsigned max_polls, int* status,
                          cudaStream_t stream) {
  if (world > MAX_RANKS) return FSB_ERR_TOO_LARGE;
  wait_kernel<<<1, 32, 0, stream>>>(static_cast<const uint32_t*>(my_flags), world, epoch, max_polls, status);
  return ok();
}

// descs: device array of nseg {src, dst, bytes, mode, pad} records; sources may be peer addresses.
// my_flags may be null (no wait).
FSB_API int fsb_comm_gather_pull(const void* descs, int nseg, int blocks_per_seg, const void* my_flags,
                                 int world, unsigned epoch, unsigned max_polls, int* status,
                                 cudaStream_t stream) {
  if (nseg <= 0) return FSB_OK;
  if (nseg > 65535 || world > MAX_RANKS) return FSB_ERR_TOO_LARGE;
  dim3 grid(blocks_per_seg < 1 ? 1 : blocks_per_seg, nseg);
  gather_pull_kernel<<<grid, 256, 0, stream>>>(static_cast<const SegDesc*>(descs),
                                               static_cast<const uint32_t*>(my_flags), world, epoch,
                                               max_polls, status);
  return ok();
}

// rows[r]: address of rank r's fp32 gradient row for this rank (n elements, 16-byte aligned).
// g_out may be null. With p != null the AdamW update is applied in the same pass.
// mc_row != 0: address of the row in the multicast mapping; the sum is then one in-switch load-reduce
// per 16 bytes (needs n % 4 == 0) and `rows` is not read.
static int reduce_rows_launch(const unsigned long long* rows, unsigned long long mc_row, int world, long long n,
                              float scale, float* g_out, void* p, int p_fp32, float* m, float* v, float lr,
                              float beta1, float beta2, float eps, float weight_decay, int step,
                              const void* my_flags, unsigned epoch, unsigned max_polls, int* status,
                              cudaStream_t stream) {
  if (world > MAX_RANKS) return FSB_ERR_TOO_LARGE;
  if (n <= 0) return FSB_OK;
  PeerPtrs rp;
  const bool mc = mc_row != 0;
  if (mc) {
    if ((mc_row & 15) || (n & 3)) return FSB_ERR_BAD_ARG;
    rp.p[0] = reinterpret_cast<void*>(mc_row);
  } else {
    for (int r = 0; r < world; ++r) {
      if (rows[r] & 15) return FSB_ERR_BAD_ARG;
      rp.p[r] = reinterpret_cast<void*>(rows[r]);
    }
  }
  AdamArgs a{lr, beta1, beta2, eps, weight_decay, 1.f - powf(beta1, static_cast<float>(step)),
             sqrtf(1.f - powf(beta2, static_cast<float>(step)))};
  const int grid = grid_for(n, 8);
  const uint32_t* fl = static_cast<const uint32_t*>(my_flags);
#define FSB_REDUCE_LAUNCH(PT, ADAM, MCF, PP)                                                              \
  reduce_rows_kernel<PT, ADAM, MCF><<<grid, 256, 0, stream>>>(rp, world, n, scale, g_out, PP, m, v, a, fl, \
                                                              epoch, max_polls, status)
  if (p == nullptr) {
    if (mc) FSB_REDUCE_LAUNCH(float, false, true, static_cast<float*>(nullptr));
    else FSB_REDUCE_LAUNCH(float, false, false, static_cast<float*>(nullptr));
  } else if (p_fp32) {
    if (mc) FSB_REDUCE_LAUNCH(float, true, true, static_cast<float*>(p));
    else FSB_REDUCE_LAUNCH(float, true, false, static_cast<float*>(p));
  } else {
    if (mc) FSB_REDUCE_LAUNCH(__nv_bfloat16, true, true, static_cast<__nv_bfloat16*>(p));
    else FSB_REDUCE_LAUNCH(__nv_bfloat16, true, false, static_cast<__nv_bfloat16*>(p));
  }
#undef FSB_REDUCE_LAUNCH
  return ok();
}

FSB_API int fsb_comm_reduce_rows(const unsigned long long* rows, int world, long long n, float scale,
                                 float* g_out, void* p, int p_fp32, float* m, float* v, float lr,
                                 float beta1, float beta2, float eps, float weight_decay, int step,
                                 const void* my_flags, unsigned epoch, unsigned max_polls, int* status,
                                 cudaStream_t stream) {
  return reduce_rows_launch(rows, 0ull, world, n, scale, g_out, p, p_fp32, m, v, lr, beta1, beta2, eps,
                            weight_decay, step, my_flags, epoch, max_polls, status, stream);
}

// The same reduction (+AdamW) with the W-way sum done inside the NVSwitch: `mc_row` is the address, in the
// multicast mapping of the symmetric gradient buffer, of the row every rank wrote for this rank.
FSB_API int fsb_comm_reduce_rows_mc(unsigned long long mc_row, int world, long long n, float scale,
                                    float* g_out, void* p, int p_fp32, float* m, float* v, float lr,
                                    float beta1, float beta2, float eps, float weight_decay, int step,
                                    const void* my_flags, unsigned epoch, unsigned max_polls, int* status,
                                    cudaStream_t stream) {
  if (mc_row == 0) return FSB_ERR_BAD_ARG;
  return reduce_rows_launch(nullptr, mc_row, world, n, scale, g_out, p, p_fp32, m, v, lr, beta1, beta2, eps,
                            weight_decay, step, my_flags, epoch, max_polls, status, stream);
}

// One launch that waits (bounded) on up to 64 flag rows, each for its own epoch: CTA i waits until every
// rank's entry of flag row i has reached epochs[i].
namespace {
struct WaitList {
  const uint32_t* flags[64];
  uint32_t epochs[64];
};
__global__ void wait_many_kernel(WaitList w, int world, uint32_t max_polls, int* status) {
  cta_wait_peers(w.flags[blockIdx.x], world, w.epochs[blockIdx.x], max_polls, status);
}
}  // namespace

// How this process loads kernels: 1 eager, 2 lazy, 0 unknown. Kernels that wait for a peer's flag must not
// meet lazy loading: the first launch of a kernel may need the context idle before its code can be loaded, the
// context is not idle while a wait kernel spins, and the flag it waits for may depend on that very launch on
// the peer. With CUDA_MODULE_LOADING=EAGER (read when CUDA initialises) every kernel is loaded up front.
FSB_API int fsb_module_loading_mode() {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuModuleGetLoadingMode", &p, cudaEnableDefault, &q) != cudaSuccess || p == nullptr) {
    (void)cudaGetLastError();
    return 0;
  }
  CUmoduleLoadingMode mode;
  if (reinterpret_cast<CUresult (*)(CUmoduleLoadingMode*)>(p)(&mode) != CUDA_SUCCESS) return 0;
  return mode == CU_MODULE_EAGER_LOADING ? 1 : 2;
}

FSB_API int fsb_comm_wait_many(const unsigned long long* flag_rows, const unsigned* epochs, int count, int world,
                               unsigned max_polls, int* status, cudaStream_t stream) {
  if (world > MAX_RANKS) return FSB_ERR_TOO_LARGE;
  for (int base = 0; base < count; base += 64) {
    WaitList w;
    const int c = count - base < 64 ? count - base : 64;
    for (int i = 0; i < c; ++i) {
      w.flags[i] = reinterpret_cast<const uint32_t*>(flag_rows[base + i]);
      w.epochs[i] = epochs[base + i];
    }
    wait_many_kernel<<<c, 32, 0, stream>>>(w, world, max_polls, status);
    if (cudaGetLastError() != cudaSuccess) return FSB_ERR_LAUNCH;
  }
  return FSB_OK;
}

// Copy a list of (source, destination, bytes) segments with the GPU's copy engines: one asynchronous
// device-to-device copy per segment on `stream`, in order. Sources may be peer addresses of a symmetric
// buffer; no SM takes part, so a gather issued this way does not compete with the kernels computing
// next to it. The caller orders the copies after the peers' "ready" flags with a wait launch.
FSB_API int fsb_comm_copy_segments_dma(const unsigned long long* src, const unsigned long long* dst,
                                       const long long* nbytes, int count, cudaStream_t stream) {
  for (int i = 0; i < count; ++i) {
    if (nbytes[i] <= 0) continue;
    if (cudaMemcpyAsync(reinterpret_cast<void*>(dst[i]), reinterpret_cast<const void*>(src[i]),
                        static_cast<size_t>(nbytes[i]), cudaMemcpyDefault, stream) != cudaSuccess) {
      cudaGetLastError();
      return FSB_ERR_LAUNCH;
    }
  }
  return FSB_OK;
}

// ------------------------------------------------------------------ expert-parallel row exchange, no host in the loop
// Token rows travel between a *sender layout* (this rank's (token, choice) pairs in expert-major order, every
// expert's block padded to 128 rows) and a *receiver layout* (the rows of this rank's local experts from all
// ranks, expert-major, padded to 128 rows: what the grouped GEMM reads). All sizes stay on the device: every
// rank publishes its per-expert counts and block offsets in symmetric memory, the receiver derives where each
// (source rank, local expert) run lands and publishes that table for the way back, and the rows are pulled out
// of the peers' memory by a kernel whose grid is sized for the worst case and whose CTAs stop at the real counts.
namespace {

struct EpTables {     // layout of the int32 table area at the start of every rank's symmetric payload
  int E, le, ep;
  __host__ __device__ int counts() const { return 0; }            // [E]   pairs per global expert (sender)
  __host__ __device__ int offs() const { return E; }              // [E+1] padded block offsets (sender layout)
  __host__ __device__ int recv_base() const { return 2 * E + 1; } // [ep*le] first row of (source, local expert) (receiver)
};

// Receiver set-up: wait for every rank's tables, then n / srow / drow of every (source rank s, local expert j) run,
// the receiver-side grouped-GEMM plan, the padding rows to clear, and the published recv_base table. One CTA.
__global__ void __launch_bounds__(256)
ep_receiver_setup_kernel(PeerPtrs tables, EpTables t, int me, long long cap_rows, int* __restrict__ n,
                         int* __restrict__ srow, int* __restrict__ drow, int* __restrict__ pad_lo,
                         int* __restrict__ pad_hi, int* __restrict__ plan_offs, int* __restrict__ tile_expert,
                         int* __restrict__ num_mtiles, const uint32_t* my_flags, uint32_t epoch, uint32_t max_polls,
                         int* status) {
  if (!cta_wait_peers(my_flags, t.ep, epoch, max_polls, status)) return;
  __threadfence_system();
  __shared__ int offs_s[kMaxLocalExperts + 1];
  __shared__ int tot_s[kMaxLocalExperts];
  const int pairs = t.ep * t.le;
  for (int q = threadIdx.x; q < pairs; q += blockDim.x) {
    const int s = q / t.le, j = q % t.le;
    const int* tb = static_cast<const int*>(tables.p[s]);
    n[q] = tb[t.counts() + me * t.le + j];
    srow[q] = tb[t.offs() + me * t.le + j];
  }
  __syncthreads();
  for (int j = threadIdx.x; j < t.le; j += blockDim.x) {
    int run = 0;
    for (int s = 0; s < t.ep; ++s) run += n[s * t.le + j];
    tot_s[j] = run;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    offs_s[0] = 0;
    for (int j = 0; j < t.le; ++j) offs_s[j + 1] = offs_s[j] + (tot_s[j] + 127) / 128 * 128;
    if (offs_s[t.le] > cap_rows) {
      // more rows than the receive buffer holds: report, and clamp so that no copy leaves the buffer
      atomicExch(status, FSB_ERR_TOO_LARGE);
      for (int j = 0; j <= t.le; ++j) offs_s[j] = offs_s[j] < cap_rows ? offs_s[j] : static_cast<int>(cap_rows);
    }
    *num_mtiles = offs_s[t.le] / 128;
  }
  __syncthreads();
  int* mine = static_cast<int*>(tables.p[me]);
  for (int j = threadIdx.x; j < t.le; j += blockDim.x) {
    int run = offs_s[j];
    for (int s = 0; s < t.ep; ++s) {
      const int q = s * t.le + j;
      const int room = offs_s[j + 1] - run;
      if (n[q] > room) n[q] = room > 0 ? room : 0;     // only after an overflow was reported
      drow[q] = run;
      mine[t.recv_base() + q] = run;
      run += n[q];
    }
    pad_lo[j] = run;
    pad_hi[j] = offs_s[j + 1];
  }
  for (int j = threadIdx.x; j <= t.le; j += blockDim.x) plan_offs[j] = offs_s[j];
  for (long long m = threadIdx.x; m < cap_rows / 128; m += blockDim.x) {
    const int row = static_cast<int>(m) * 128;
    int a = 0, b = t.le;
    while (a < b) {
      const int mid = (a + b) / 2;
      if (offs_s[mid + 1] > row) b = mid; else a = mid + 1;
    }
    tile_expert[m] = a < t.le ? a : t.le - 1;
  }
}

// Sender set-up for the way back: wait until every receiver has published recv_base, then for every
// (destination rank r, its local expert j): n = my count, srow = r's row of my run, drow = my block's row.
__global__ void __launch_bounds__(256)
ep_sender_setup_kernel(PeerPtrs tables, EpTables t, int me, long long cap_rows, int* __restrict__ n,
                       int* __restrict__ srow, int* __restrict__ drow, const uint32_t* my_flags, uint32_t epoch,
                       uint32_t max_polls, int* status) {
  if (!cta_wait_peers(my_flags, t.ep, epoch, max_polls, status)) return;
  __threadfence_system();
  const int* mine = static_cast<const int*>(tables.p[me]);
  for (int q = threadIdx.x; q < t.ep * t.le; q += blockDim.x) {
    const int r = q / t.le, j = q % t.le;
    const int* tb = static_cast<const int*>(tables.p[r]);
    const int base = tb[t.recv_base() + me * t.le + j];
    // a receiver that overflowed (and reported it) clamped its runs: never read past the end of its row area
    const long long room = cap_rows - base;
    const int cnt = mine[t.counts() + q];
    n[q] = (base < 0 || room <= 0) ? 0 : (cnt < room ? cnt : static_cast<int>(room));
    srow[q] = base < 0 ? 0 : base;
    drow[q] = mine[t.offs() + q];
  }
}

// Pull runs of rows: run q copies n[q] rows from peer q / le's area (row srow[q]) to row drow[q] of `dst`.
// blockIdx.y >= pairs clears the padding rows [pad_lo[j], pad_hi[j]) of expert block j (pad_lo may be null).
__global__ void __launch_bounds__(256)
ep_pull_rows_kernel(PeerPtrs area, const int* __restrict__ n, const int* __restrict__ srow,
                    const int* __restrict__ drow, const int* __restrict__ pad_lo, const int* __restrict__ pad_hi,
                    uint8_t* __restrict__ dst, long long row_bytes, int pairs, int le, const uint32_t* my_flags,
                    int world, uint32_t epoch, uint32_t max_polls, int* status) {
  if (my_flags != nullptr && !cta_wait_peers(my_flags, world, epoch, max_polls, status)) return;
  const int q = blockIdx.y;
  const long long vec = row_bytes / 16;
  if (q >= pairs) {
    if (pad_lo == nullptr) return;
    const int j = q - pairs;
    const long long lo = pad_lo[j], hi = pad_hi[j];
    uint4* d = reinterpret_cast<uint4*>(dst + lo * row_bytes);
    const uint4 z = make_uint4(0, 0, 0, 0);
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < (hi - lo) * vec;
         i += static_cast<long long>(gridDim.x) * blockDim.x)
      d[i] = z;
    return;
  }
  const long long rows = n[q];
  if (rows <= 0) return;
  const uint4* s = reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(area.p[q / le]) + srow[q] * row_bytes);
  uint4* d = reinterpret_cast<uint4*>(dst + drow[q] * row_bytes);
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < rows * vec;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    d[i] = s[i];
}

}  // namespace

// tables[r]: address of rank r's int32 table area. Outputs are local device int32 arrays (n, srow, drow of
// ep*le runs; pad_lo / pad_hi of le blocks; the grouped-GEMM plan of the receive layout).
FSB_API int fsb_ep_receiver_setup(const unsigned long long* tables, int E, int le, int ep, int me,
                                  long long cap_rows, int* n, int* srow, int* drow, int* pad_lo, int* pad_hi,
                                  int* plan_offs, int* tile_expert, int* num_mtiles, const void* my_flags,
                                  unsigned epoch, unsigned max_polls, int* status, cudaStream_t stream) {
  if (ep > MAX_RANKS || le > kMaxLocalExperts || E != ep * le || cap_rows % 128 != 0) return FSB_ERR_BAD_ARG;
  PeerPtrs tp;
  for (int r = 0; r < ep; ++r) tp.p[r] = reinterpret_cast<void*>(tables[r]);
  ep_receiver_setup_kernel<<<1, 256, 0, stream>>>(tp, EpTables{E, le, ep}, me, cap_rows, n, srow, drow, pad_lo,
                                                   pad_hi, plan_offs, tile_expert, num_mtiles,
                                                   static_cast<const uint32_t*>(my_flags), epoch, max_polls, status);
  return ok();
}

FSB_API int fsb_ep_sender_setup(const unsigned long long* tables, int E, int le, int ep, int me, long long cap_rows,
                                int* n, int* srow, int* drow, const void* my_flags, unsigned epoch,
                                unsigned max_polls, int* status, cudaStream_t stream) {
  if (ep > MAX_RANKS || le > kMaxLocalExperts || E != ep * le || cap_rows <= 0) return FSB_ERR_BAD_ARG;
  PeerPtrs tp;
  for (int r = 0; r < ep; ++r) tp.p[r] = reinterpret_cast<void*>(tables[r]);
  ep_sender_setup_kernel<<<1, 256, 0, stream>>>(tp, EpTables{E, le, ep}, me, cap_rows, n, srow, drow,
                                                 static_cast<const uint32_t*>(my_flags), epoch, max_polls, status);
  return ok();
}

// area[r]: address of rank r's row area (rows of row_bytes, a multiple of 16). my_flags may be null (no wait).
FSB_API int fsb_ep_pull_rows(const unsigned long long* area, const int* n, const int* srow, const int* drow,
                             const int* pad_lo, const int* pad_hi, void* dst, long long row_bytes, int ep, int le,
                             int blocks_per_run, const void* my_flags, unsigned epoch, unsigned max_polls,
                             int* status, cudaStream_t stream) {
  if (ep > MAX_RANKS || row_bytes % 16 != 0 || (reinterpret_cast<uintptr_t>(dst) & 15)) return FSB_ERR_BAD_ARG;
  PeerPtrs ap;
  for (int r = 0; r < ep; ++r) {
    if (area[r] & 15) return FSB_ERR_BAD_ARG;
    ap.p[r] = reinterpret_cast<void*>(area[r]);
  }
  const int pairs = ep * le;
  dim3 grid(blocks_per_run < 1 ? 1 : blocks_per_run, pairs + (pad_lo != nullptr ? le : 0));
  ep_pull_rows_kernel<<<grid, 256, 0, stream>>>(ap, n, srow, drow, pad_lo, pad_hi, static_cast<uint8_t*>(dst),
                                                row_bytes, pairs, le, static_cast<const uint32_t*>(my_flags), ep,
                                                epoch, max_polls, status);
  return ok();
}
