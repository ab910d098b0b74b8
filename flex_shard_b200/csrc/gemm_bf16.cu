// Persistent bf16 GEMM for sm_100a: TMA-fed shared-memory ring, tcgen05.mma
// issued by one thread, fp32 accumulators double-buffered in TMEM, epilogue
// warps draining one accumulator while the tensor core fills the other.
//
//   D[M,N] = alpha * (A[M,K] . B[N,K]^T) + beta * C[M,N]  (+ D when accumulate)
//
// A and B may each be stored K-major (row = M/N index, K contiguous) or
// MN-major (row = K index, M/N contiguous), which covers the three GEMMs of a
// linear layer without a transpose pass:
//   forward  y  = x W^T   : A = x  (K-major),  B = W  (K-major)
//   dgrad    dx = dy W    : A = dy (K-major),  B = W  (MN-major)
//   wgrad    dW = dy^T x  : A = dy (MN-major), B = x  (MN-major)
// D and C are row-major, bf16 or fp32.
//
// Warp roles (192 threads): warp 0 = TMA producer, warp 1 = TMEM owner + MMA
// issuer, warps 2..5 = epilogue (one TMEM lane quarter each).
#include "common.cuh"
#include <stdio.h>

namespace {

using namespace fsb;

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;          // 64 bf16 = one 128-byte swizzle atom
constexpr int UMMA_K = 16;
constexpr int STAGES = 4;
constexpr int A_STAGE_BYTES = BM * BK * 2;  // 16 KB
constexpr int B_STAGE_BYTES = BN * BK * 2;  // 32 KB
constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int TMEM_COLS = 512;              // two 256-column accumulators
constexpr int GROUP_M = 8;                  // tile rasterisation group
constexpr int NUM_THREADS = 192;
constexpr int EPI_STAGE_BYTES = 4 * 32 * 33 * 4;  // per epilogue warp: a padded 32x32 fp32 transpose tile
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align slack*/ + 256 /*barriers*/ + EPI_STAGE_BYTES;

struct GemmArgs {
  int M, N, K;
  int a_mn, b_mn;
  void* d;
  long long ldd;
  int d_fp32;
  const void* c;
  long long ldc;
  int c_fp32;
  float alpha, beta;
  int accumulate;
  int upper_only;     // two-SM kernel, M == N: compute only the 256x256 tiles on or above the diagonal
  // When d_block_rows > 0, D is cut into blocks of that many rows and block i starts at
  // element offset i * d_block_stride (the [world, rows/world, N] rows of a reduce-scatter
  // send buffer), so a weight gradient can be written straight into its reduction layout.
  long long d_block_rows, d_block_stride;
  // With d_peer_n > 0 block i of D starts at d_peer[i] instead (another GPU's memory mapped over
  // NVLink): the epilogue's stores ARE the all-to-all leg of a reduce-scatter.
  void* d_peer[16];
  int d_peer_n;
  int d_peer_remote;   // the blocks are in other GPUs' memory: store whole 128-byte row segments
  // Grouped (mixture-of-experts) modes; rows of every group start on a multiple of 128 and are
  // padded with zero rows to a multiple of 128.
  //   1: grouped rows  - A [R, K]; m-tile t belongs to expert tile_expert[t] and multiplies that
  //      expert's B slice (b_group_rows rows of B per expert); *num_mtiles m-tiles are valid
  //   2: grouped K     - D [E, M, N] = A_e^T-style products over each expert's row range
  //      [group_offs[e], group_offs[e+1]) of the MN-major operands A [R, M] and B [R, N]
  int group_mode;
  int num_groups;
  const int* tile_expert;
  const int* num_mtiles;
  const int* group_offs;
  long long b_group_rows;
  int* status;
};

struct TileInfo {
  int tm, tn;
  int num_kb;
  int k_off;          // added to the K coordinate of both operands (mode 2)
  int b_row_off;      // added to B's N coordinate (K-major B) or K coordinate (MN-major B) (mode 1)
  long long d_row_off;
  bool valid;
};

// All-gather fused into the GEMM: `n_stagers` CTAs of the grid pull the weight's row shards from
// the peers' memory (NVLink) into the local gathered buffer, 16 KB pieces through a shared-memory
// ring of bulk copies, in the order the GEMM consumes them; the GEMM CTAs wait per 256-row chunk.
constexpr int AG_PIECE = 16384;
constexpr int AG_RING = 11;          // 176 KB of the CTA's shared memory
constexpr int AG_LAG = 3;            // store groups allowed in flight before completion is published
constexpr int AG_MAX_RANKS = 16;
struct AgArgs {
  const uint8_t* peer[AG_MAX_RANKS];  // peer[r]: rank r's shard of the weight (shard_bytes each)
  uint8_t* local;                     // gathered weight [N, K] bf16, row-major, ld == K
  long long shard_bytes, total_bytes, chunk_bytes;  // chunk = BN rows
  int* counters;                      // [tiles_n] pieces landed per chunk (monotonic across calls)
  int call_index;                     // 1-based number of this call for these counters
  int n_stagers;
  const uint32_t* peer_flags;         // this rank's flag row: peers' shards are valid from `epoch` on
  int world;
  uint32_t epoch, max_polls;
};

__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void bulk_store(void* gdst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
               ::"l"(gdst), "r"(smem_u32(smem_src)), "r"(bytes) : "memory");
}

__device__ __forceinline__ void tile_coords_nmajor(int tile, int tiles_m, int& tm, int& tn) {
  tn = tile / tiles_m;
  tm = tile % tiles_m;
}

__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int& tm, int& tn) {
  const int per_group = GROUP_M * tiles_n;
  const int group = tile / per_group;
  const int first_m = group * GROUP_M;
  const int rows = min(tiles_m - first_m, GROUP_M);
  const int in_group = tile - group * per_group;
  tm = first_m + in_group % rows;
  tn = in_group / rows;
}

template <bool AG>
__device__ __forceinline__ TileInfo get_tile(const GemmArgs& args, int tile, int tiles_m, int tiles_n,
                                             int num_kb_full) {
  TileInfo t;
  t.num_kb = num_kb_full;
  t.k_off = 0;
  t.b_row_off = 0;
  t.d_row_off = 0;
  t.valid = true;
  if (AG) {
    tile_coords_nmajor(tile, tiles_m, t.tm, t.tn);
  } else if (args.group_mode == 2) {
    const int per = tiles_m * tiles_n;
    const int e = tile / per;
    tile_coords(tile - e * per, tiles_m, tiles_n, t.tm, t.tn);
    const int r0 = args.group_offs[e], r1 = args.group_offs[e + 1];
    t.k_off = r0;
    t.num_kb = (r1 - r0 + BK - 1) / BK;
    t.d_row_off = static_cast<long long>(e) * args.M;
  } else {
    tile_coords(tile, tiles_m, tiles_n, t.tm, t.tn);
    if (args.group_mode == 1) {
      t.valid = t.tm < *args.num_mtiles;
      if (t.valid) t.b_row_off = args.tile_expert[t.tm] * static_cast<int>(args.b_group_rows);
    }
  }
  return t;
}

// Epilogue of one 128 x 256 accumulator tile: the calling warp owns TMEM lanes [32*quarter, +32)
// (t_row = TMEM address of its lane quarter, column 0 of the accumulator) = rows
// tm*128 + 32*quarter + lane of D. `stg` is the warp's padded 32x32 fp32 staging tile.
__device__ __forceinline__ void store_tile(const GemmArgs& args, long long d_row_off, int tm, int tn,
                                           uint32_t t_row, float* stg, int quarter, int lane) {
  const long long row = static_cast<long long>(tm) * BM + quarter * 32 + lane;
  const bool row_ok = row < args.M;
  long long d_off = args.d_block_rows > 0
                        ? (row / args.d_block_rows) * args.d_block_stride +
                              (row % args.d_block_rows) * args.ldd
                        : (d_row_off + row) * args.ldd;
  void* d_base = args.d;
  if (args.d_peer_n > 0 && row_ok) {
    d_base = args.d_peer[row / args.d_block_rows];
    d_off = (row % args.d_block_rows) * args.ldd;
  }
#pragma unroll 1
  for (int c0 = 0; c0 < BN; c0 += 32) {
    const int col = tn * BN + c0;
    if (col >= args.N) break;  // uniform across the warp
    uint32_t r[32];
    tmem_ld_32x32(t_row + c0, r);
    tmem_ld_wait();
    if (args.d_peer_remote && args.d_peer_n > 0 && args.d_fp32 && !args.accumulate && args.c == nullptr && col + 32 <= args.N) {
      // Rows of this tile live in other GPUs' memory: transpose the warp's 32x32 block through
      // shared memory so that every store instruction writes one full 128-byte row segment
      // (NVLink moves whole lines efficiently, scattered 16-byte pieces poorly).
#pragma unroll
      for (int i = 0; i < 32; ++i) stg[lane * 33 + i] = __uint_as_float(r[i]) * args.alpha;
      __syncwarp();
      const long long row0 = static_cast<long long>(tm) * BM + quarter * 32;
#pragma unroll 4
      for (int rr = 0; rr < 32; ++rr) {
        const long long gr = row0 + rr;
        if (gr < args.M) {
          float* base = static_cast<float*>(args.d_peer[gr / args.d_block_rows]) +
                        (gr % args.d_block_rows) * args.ldd + col;
          base[lane] = stg[rr * 33 + lane];
        }
      }
      __syncwarp();
      continue;
    }
    if (row_ok) {
      float v[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) * args.alpha;
      const bool full = (col + 32 <= args.N);
      if (args.c != nullptr) {
        if (args.c_fp32) {
          const float* cp = static_cast<const float*>(args.c) + (d_row_off + row) * args.ldc + col;
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (full || col + i < args.N) v[i] += args.beta * cp[i];
        } else {
          const __nv_bfloat16* cp =
              static_cast<const __nv_bfloat16*>(args.c) + (d_row_off + row) * args.ldc + col;
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (full || col + i < args.N) v[i] += args.beta * __bfloat162float(cp[i]);
        }
      }
      if (args.d_fp32) {
        float* dp = static_cast<float*>(d_base) + d_off + col;
        if (full && (args.ldd % 4 == 0) && (args.d_block_stride % 4 == 0)) {
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            float4 o = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
            if (args.accumulate) {
              const float4 old = *reinterpret_cast<const float4*>(dp + i);
              o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
            }
            *reinterpret_cast<float4*>(dp + i) = o;
          }
        } else {
          for (int i = 0; i < 32; ++i)
            if (col + i < args.N) dp[i] = args.accumulate ? dp[i] + v[i] : v[i];
        }
      } else {
        __nv_bfloat16* dp = static_cast<__nv_bfloat16*>(d_base) + d_off + col;
        if (full && (args.ldd % 8 == 0) && (args.d_block_stride % 8 == 0)) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            if (args.accumulate) {
              const uint4 old = *reinterpret_cast<const uint4*>(dp + i);
              const __nv_bfloat162* ob = reinterpret_cast<const __nv_bfloat162*>(&old);
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const float2 f = __bfloat1622float2(ob[j]);
                v[i + 2 * j] += f.x;
                v[i + 2 * j + 1] += f.y;
              }
            }
            uint4 o;
            o.x = pack_bf16x2(v[i], v[i + 1]);
            o.y = pack_bf16x2(v[i + 2], v[i + 3]);
            o.z = pack_bf16x2(v[i + 4], v[i + 5]);
            o.w = pack_bf16x2(v[i + 6], v[i + 7]);
            *reinterpret_cast<uint4*>(dp + i) = o;
          }
        } else {
          for (int i = 0; i < 32; ++i)
            if (col + i < args.N) {
              const float o = args.accumulate ? __bfloat162float(dp[i]) + v[i] : v[i];
              dp[i] = __float2bfloat16(o);
            }
        }
      }
    }
  }
}

template <bool AG>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                 const GemmArgs args, const AgArgs ag) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* full_bar = bars;                    // [STAGES]
  uint64_t* empty_bar = bars + STAGES;          // [STAGES]
  uint64_t* tmem_full = bars + 2 * STAGES;      // [2]
  uint64_t* tmem_empty = bars + 2 * STAGES + 2; // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tiles_m = (args.M + BM - 1) / BM;
  const int tiles_n = (args.N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n * (args.group_mode == 2 ? args.num_groups : 1);
  const int num_kb = (args.K + BK - 1) / BK;
  const bool stager = AG && static_cast<int>(blockIdx.x) < ag.n_stagers;
  const int tile0 = AG ? static_cast<int>(blockIdx.x) - ag.n_stagers : static_cast<int>(blockIdx.x);
  const int tile_step = AG ? static_cast<int>(gridDim.x) - ag.n_stagers : static_cast<int>(gridDim.x);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tmem_full[i], 1);
      mbar_init(&tmem_empty[i], 4);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1 && !stager) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = stager ? 0u : *tmem_slot;

  if (stager) {
    // ------------------------------------------------------------ all-gather stager CTA
    if constexpr (AG) {
      if (threadIdx.x == 0) {
        uint64_t* ring_bar = bars + 2 * STAGES + 8;  // [AG_RING], past the GEMM's barriers
        for (int i = 0; i < AG_RING; ++i) mbar_init(&ring_bar[i], 1);
        mbar_fence_init();
        bool ok = true;
        // peers' shards must be valid (their optimizer step of this epoch has been published)
        for (int r = 0; r < ag.world && ok; ++r) {
          uint32_t polls = 0;
          while (static_cast<int32_t>(ld_acquire_sys_u32(ag.peer_flags + r) - ag.epoch) < 0) {
            if (++polls > ag.max_polls) {
              ok = false;
              break;
            }
            if (polls > 64) __nanosleep(200);
          }
        }
        if (!ok) {
          atomicExch(args.status, FSB_ERR_WAIT_TIMEOUT_PEER);
        } else {
          // Work list of this stager: inside every 256-row chunk a contiguous run of pieces, chunks in
          // the order the GEMM consumes them. Completion is published once per (stager, chunk).
          const int S = ag.n_stagers, me = blockIdx.x;
          const long long n_chunks = (ag.total_bytes + ag.chunk_bytes - 1) / ag.chunk_bytes;
          auto chunk_pieces = [&](long long c) {
            long long hi = (c + 1) * ag.chunk_bytes;
            if (hi > ag.total_bytes) hi = ag.total_bytes;
            return (hi - c * ag.chunk_bytes + AG_PIECE - 1) / AG_PIECE;
          };
          auto my_lo = [&](long long c) { return chunk_pieces(c) * me / S; };
          auto my_hi = [&](long long c) { return chunk_pieces(c) * (me + 1) / S; };
          // iterator over (chunk, piece) pairs of this stager, used twice: for loads (ahead) and stores
          struct It { long long c, p; };
          auto advance = [&](It& it) {
            ++it.p;
            while (it.c < n_chunks && it.p >= my_hi(it.c)) {
              ++it.c;
              if (it.c < n_chunks) it.p = my_lo(it.c);
            }
          };
          auto first = [&]() {
            It it{0, my_lo(0)};
            while (it.c < n_chunks && it.p >= my_hi(it.c)) {
              ++it.c;
              if (it.c < n_chunks) it.p = my_lo(it.c);
            }
            return it;
          };
          auto off_of = [&](const It& it) { return it.c * ag.chunk_bytes + it.p * static_cast<long long>(AG_PIECE); };
          auto len_of = [&](const It& it) {
            const long long rem = ag.total_bytes - off_of(it);
            return static_cast<uint32_t>(rem < AG_PIECE ? rem : AG_PIECE);
          };
          long long n_loaded = 0, n_stored = 0;
          It ld = first(), st = first();
          auto issue_load = [&]() {
            const long long off = off_of(ld);
            const int owner = static_cast<int>(off / ag.shard_bytes);
            const int slot = static_cast<int>(n_loaded % AG_RING);
            mbar_expect_tx(&ring_bar[slot], len_of(ld));
            bulk_load(smem + slot * AG_PIECE, ag.peer[owner] + (off - owner * ag.shard_bytes), len_of(ld),
                      &ring_bar[slot]);
            ++n_loaded;
            advance(ld);
          };
          const long long ahead = AG_RING - AG_LAG - 1;
          while (ld.c < n_chunks && n_loaded < ahead) issue_load();
          while (st.c < n_chunks && ok) {
            const int slot = static_cast<int>(n_stored % AG_RING);
            if (!mbar_wait(&ring_bar[slot], static_cast<uint32_t>(n_stored / AG_RING) & 1, abort_flag)) {
              atomicExch(args.status, FSB_ERR_WAIT_TIMEOUT_FULL);
              ok = false;
              break;
            }
            bulk_store(ag.local + off_of(st), smem + slot * AG_PIECE, len_of(st));
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            ++n_stored;
            const long long c_done = st.c;
            const long long pieces_in_chunk = my_hi(c_done) - my_lo(c_done);
            advance(st);
            if (st.c != c_done) {
              // last piece of this chunk: wait for the stores to land, then publish them
              asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
              asm volatile("fence.proxy.async;" ::: "memory");
              __threadfence();
              atomicAdd(ag.counters + static_cast<int>(c_done), static_cast<int>(pieces_in_chunk));
            } else {
              // the slot that the next load will reuse must have been read by its store
              asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(AG_LAG) : "memory");
            }
            if (ld.c < n_chunks) issue_load();
          }
          asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
          if (!ok) {
            // A ring wait ran out: tell the rest of the CTA, then give every load that was issued but not
            // consumed a (bounded) chance to land before the CTA may exit, so that no bulk copy is still
            // writing this CTA's shared memory afterwards. The GEMM CTAs give up on their chunk waits by
            // their own bounds.
            *abort_flag = 1;
            for (long long i = n_stored; i < n_loaded; ++i) {
              const int slot = static_cast<int>(i % AG_RING);
              const uint32_t parity = static_cast<uint32_t>(i / AG_RING) & 1;
              for (uint32_t t = 0; t < kSpinFast * 16u; ++t)
                if (mbar_try_wait_hint(&ring_bar[slot], parity, kWaitHintNs)) break;
            }
          }
        }
      }
    }
  } else if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&map_a);
      tma_prefetch_desc(&map_b);
      uint32_t it = 0;
      bool ok = true;
      int ready_tn = -1;
      for (int tile = tile0; tile < num_tiles && ok; tile += tile_step) {
        const TileInfo ti = get_tile<AG>(args, tile, tiles_m, tiles_n, num_kb);
        if (!ti.valid || ti.num_kb == 0) continue;
        const int tm = ti.tm, tn = ti.tn;
        const int m0 = tm * BM, n0 = tn * BN;
        if (AG && tn != ready_tn) {
          // wait until every piece of this 256-row chunk of the weight has landed locally
          const long long lo = static_cast<long long>(tn) * ag.chunk_bytes;
          long long hi = lo + ag.chunk_bytes;
          if (hi > ag.total_bytes) hi = ag.total_bytes;
          const int pieces = static_cast<int>((hi - lo + AG_PIECE - 1) / AG_PIECE);
          const int target = pieces * ag.call_index;
          uint32_t polls = 0;
          while (ld_acquire_gpu(ag.counters + tn) < target) {
            if (++polls > ag.max_polls || *abort_flag) {
              atomicExch(args.status, FSB_ERR_WAIT_TIMEOUT_PEER);
              *abort_flag = 1;
              ok = false;
              break;
            }
            if (polls > 32) __nanosleep(100);
          }
          if (!ok) break;
          asm volatile("fence.proxy.async;" ::: "memory");  // generic-proxy flag -> async-proxy (TMA) reads
          ready_tn = tn;
        }
        for (int kb = 0; kb < ti.num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&empty_bar[s], ph ^ 1, abort_flag)) {
            atomicExch(args.status, FSB_ERR_WAIT_TIMEOUT_EMPTY);
            *abort_flag = 1;
            ok = false;
            break;
          }
          uint8_t* sa = smem + s * STAGE_BYTES;
          uint8_t* sb = sa + A_STAGE_BYTES;
          mbar_expect_tx(&full_bar[s], STAGE_BYTES);
          const int k0 = kb * BK + ti.k_off;
          if (!args.a_mn) {
            tma_load_2d(sa, &map_a, &full_bar[s], k0, m0);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)
              tma_load_2d(sa + j * 8192, &map_a, &full_bar[s], m0 + 64 * j, k0);
          }
          if (!args.b_mn) {
            tma_load_2d(sb, &map_b, &full_bar[s], k0, n0 + ti.b_row_off);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_2d(sb + j * 8192, &map_b, &full_bar[s], n0 + 64 * j, k0 + ti.b_row_off);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    // The whole warp walks the loop (waits and descriptor arithmetic stay warp-uniform); one elected
    // lane issues the tcgen05 instructions.
    {
      const uint32_t idesc = make_idesc(BM, BN, 1, 1, args.a_mn ? 1u : 0u, args.b_mn ? 1u : 0u);
      // K-major: 8-row groups 1024 B apart, K step of 16 elements = 32 B inside the atom.
      // MN-major: 64-wide MN groups 8192 B apart (LBO), 8-deep K groups 1024 B apart (SBO),
      //           K step of 16 = two K groups = 2048 B.
      const uint32_t a_lbo = args.a_mn ? 8192u : 16u, b_lbo = args.b_mn ? 8192u : 16u;
      const uint32_t a_kstep = (args.a_mn ? 2048u : 32u) >> 4, b_kstep = (args.b_mn ? 2048u : 32u) >> 4;
      uint32_t it = 0, local_tile = 0;
      bool ok = true;
      for (int tile = tile0; tile < num_tiles && ok; tile += tile_step) {
        const TileInfo ti = get_tile<AG>(args, tile, tiles_m, tiles_n, num_kb);
        if (!ti.valid || ti.num_kb == 0) continue;
        const uint32_t acc = local_tile & 1;
        const uint32_t acc_ph = (local_tile >> 1) & 1;
        ++local_tile;
        if (!mbar_wait(&tmem_empty[acc], acc_ph ^ 1, abort_flag)) {
          if (lane == 0) {
            atomicExch(args.status, FSB_ERR_WAIT_TIMEOUT_TMEM_EMPTY);
            *abort_flag = 1;
          }
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < ti.num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&full_bar[s], ph, abort_flag)) {
            if (lane == 0) {
              atomicExch(args.status, FSB_ERR_WAIT_TIMEOUT_FULL);
              *abort_flag = 1;
            }
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * STAGE_BYTES);
          const uint64_t da = make_smem_desc_sw128(sa, a_lbo, 1024);
          const uint64_t db = make_smem_desc_sw128(sa + A_STAGE_BYTES, b_lbo, 1024);
          if (elect_one()) {
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k)
              umma_f16(d_tmem, da + k * a_kstep, db + k * b_kstep, idesc, (kb | k) != 0 ? 1u : 0u);
            umma_commit(&empty_bar[s]);  // stage is free once these MMAs have read it
          }
          __syncwarp();
        }
        if (ok) {
          if (elect_one()) umma_commit(&tmem_full[acc]);
          __syncwarp();
        }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int quarter = warp & 3;  // TMEM lanes [32*quarter, 32*quarter+32)
    uint32_t local_tile = 0;
    for (int tile = tile0; tile < num_tiles; tile += tile_step) {
      const TileInfo ti = get_tile<AG>(args, tile, tiles_m, tiles_n, num_kb);
      if (!ti.valid) continue;
      const int tm = ti.tm, tn = ti.tn;
      const long long row = static_cast<long long>(tm) * BM + quarter * 32 + lane;
      const bool row_ok = row < args.M;
      if (ti.num_kb == 0) {
        // an empty group contributes nothing: its output tile is zero (or left alone when accumulating)
        if (row_ok && !args.accumulate) {
          for (int c = tn * BN; c < min(args.N, tn * BN + BN); ++c) {
            const long long o = (ti.d_row_off + row) * args.ldd + c;
            if (args.d_fp32) static_cast<float*>(args.d)[o] = 0.f;
            else static_cast<__nv_bfloat16*>(args.d)[o] = __float2bfloat16(0.f);
          }
        }
        continue;
      }
      const uint32_t acc = local_tile & 1;
      const uint32_t acc_ph = (local_tile >> 1) & 1;
      ++local_tile;
      if (!mbar_wait(&tmem_full[acc], acc_ph, abort_flag)) {
        if (lane == 0) {
          atomicExch(args.status, FSB_ERR_WAIT_TIMEOUT_TMEM_FULL);
          *abort_flag = 1;
        }
        break;
      }
      tc_fence_after();
      store_tile(args, ti.d_row_off, tm, tn, tmem_base + acc * BN + (static_cast<uint32_t>(quarter * 32) << 16),
                 reinterpret_cast<float*>(smem + STAGES * STAGE_BYTES + 256) + (warp - 2) * 32 * 33, quarter, lane);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[acc]);
    }
  }

  // Common exit: every loop above is bounded, so all warps arrive here.
  tc_fence_before();
  __syncthreads();
  if (warp == 1 && !stager) {
    if (*abort_flag) {
      // Give copies that were already issued time to land before the CTA's
      // shared memory and TMEM go away.
      const unsigned long long t0 = clock64();
      while (clock64() - t0 < 2000000ull) {
      }
    }
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------------------
// Two-SM variant for dense GEMMs: a cluster of two CTAs (one SM pair) owns a 256 x 256 tile of D.
// CTA r of the pair loads rows [128 r, 128 r + 128) of the A tile and rows [128 r, +128) of the B
// tile into its own shared memory; one thread of CTA 0 issues tcgen05.mma.cta_group::2, which
// reads both CTAs' operands and accumulates D rows [128 r, +128) x 256 columns into CTA r's TMEM.
// Per SM and per 16-deep step the tensor core reads 4 KB of A and 4 KB of B instead of 4 KB + 8 KB,
// which takes the operand reads off the shared-memory bandwidth limit, and each SM's ring holds
// 6 x 64-deep stages instead of 4.
// Signals that cross the pair: TMA completion bytes of both CTAs land on CTA 0's `full` barrier;
// tcgen05.commit arrives on the `empty` / `tmem_full` barriers of both CTAs; the epilogue warps of
// both CTAs arrive on CTA 0's `tmem_empty` barrier. Every wait is bounded; a CTA that gives up
// still walks to the cluster barrier at the end, so its peer is never left alone.
constexpr int BN_HALF = 128;                       // B rows per CTA
constexpr int STAGES2 = 6;
constexpr int B2_STAGE_BYTES = BN_HALF * BK * 2;   // 16 KB
constexpr int STAGE2_BYTES = A_STAGE_BYTES + B2_STAGE_BYTES;
constexpr int SMEM2_BYTES = STAGES2 * STAGE2_BYTES + 1024 + 256 + EPI_STAGE_BYTES;

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of the same shared-memory location in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA tile load of the executing CTA whose completion bytes are counted on a barrier that may live in
// the peer CTA of the pair (no fan-out of the data: each CTA fetches its own tiles).
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, uint32_t bar_cluster_addr,
                                                 int32_t c0, int32_t c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void umma_f16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                              uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// One arrival on the barrier at `cluster_addr` (own or peer CTA) once every MMA issued so far has retired.
__device__ __forceinline__ void umma_commit_pair(uint32_t cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_addr)
               : "memory");
}

// When the rows of D live in several GPUs' memory (row block i belongs to rank i), consecutive tiles
// are dealt round-robin over the row blocks, so the CTAs that run at the same time write to all
// owners at once instead of bursting into one NVLink destination after the other.
__device__ __forceinline__ int spread_over_row_blocks(int tm, int tiles_m, int nblk) {
  const int per = tiles_m / nblk;
  return (tm % nblk) * per + tm / nblk;
}

// Tile `t` of the upper triangle (diagonal included) of a T x T tile grid, row by row.
__device__ __forceinline__ void upper_tile_coords(int t, int T, int& tm, int& tn) {
  tm = 0;
  while (t >= T - tm) {
    t -= T - tm;
    ++tm;
  }
  tn = tm + t;
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
gemm_bf16_2sm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                     const GemmArgs args) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES2 * STAGE2_BYTES);
  uint64_t* full_bar = bars;                      // [STAGES2]  used in CTA 0
  uint64_t* empty_bar = bars + STAGES2;           // [STAGES2]  one per CTA
  uint64_t* tmem_full = bars + 2 * STAGES2;       // [2]        one per CTA
  uint64_t* tmem_empty = bars + 2 * STAGES2 + 2;  // [2]        used in CTA 0 (8 arrivals: 4 warps x 2 CTAs)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES2 + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int tiles_m = (args.M + 2 * BM - 1) / (2 * BM);   // 256-row tiles
  const int tiles_n = (args.N + BN - 1) / BN;
  const int num_tiles = args.upper_only ? tiles_m * (tiles_m + 1) / 2 : tiles_m * tiles_n;
  const int num_kb = (args.K + BK - 1) / BK;
  const int tile0 = static_cast<int>(blockIdx.x >> 1);
  const int tile_step = static_cast<int>(gridDim.x >> 1);
  const bool spread = args.d_peer_remote && args.d_peer_n > 1 && args.d_block_rows % (2 * BM) == 0 &&
                      static_cast<long long>(tiles_m) * (2 * BM) == args.d_block_rows * args.d_peer_n;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES2; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tmem_full[i], 1);
      mbar_init(&tmem_empty[i], 8);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();   // the peer's barriers are initialised before anything is signalled across the pair
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      tma_prefetch_desc(&map_a);
      tma_prefetch_desc(&map_b);
      uint32_t it = 0;
      bool ok = true;
      for (int tile = tile0; tile < num_tiles && ok; tile += tile_step) {
        int tm2, tn;
        if (args.upper_only) {
          upper_tile_coords(tile, tiles_m, tm2, tn);
        } else {
          tile_coords(tile, tiles_m, tiles_n, tm2, tn);
          if (spread) tm2 = spread_over_row_blocks(tm2, tiles_m, args.d_peer_n);
        }
        const int m0 = tm2 * 2 * BM + static_cast<int>(rank) * BM;
        const int n0 = tn * BN + static_cast<int>(rank) * BN_HALF;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % STAGES2;
          const uint32_t ph = (it / STAGES2) & 1;
          if (!mbar_wait(&empty_bar[s], ph ^ 1, abort_flag)) {
            atomicExch(args.status, FSB_ERR_WAIT_TIMEOUT_EMPTY);
            *abort_flag = 1;
            ok = false;
            break;
          }
          uint8_t* sa = smem + s * STAGE2_BYTES;
          uint8_t* sb = sa + A_STAGE_BYTES;
          const uint32_t full0 = map_to_cta(smem_u32(&full_bar[s]), 0);
          if (rank == 0) mbar_expect_tx(&full_bar[s], 2 * STAGE2_BYTES);   // the bytes of both CTAs
          const int k0 = kb * BK;
          if (!args.a_mn) {
            tma_load_2d_pair(sa, &map_a, full0, k0, m0);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_2d_pair(sa + j * 8192, &map_a, full0, m0 + 64 * j, k0);
          }
          if (!args.b_mn) {
            tma_load_2d_pair(sb, &map_b, full0, k0, n0);
          } else {
#pragma unroll
            for (int j = 0; j < BN_HALF / 64; ++j) tma_load_2d_pair(sb + j * 8192, &map_b, full0, n0 + 64 * j, k0);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (CTA 0 only)
    if (rank == 0) {
      const uint32_t idesc = make_idesc(2 * BM, BN, 1, 1, args.a_mn ? 1u : 0u, args.b_mn ? 1u : 0u);
      const uint32_t a_lbo = args.a_mn ? 8192u : 16u, b_lbo = args.b_mn ? 8192u : 16u;
      const uint32_t a_kstep = (args.a_mn ? 2048u : 32u) >> 4, b_kstep = (args.b_mn ? 2048u : 32u) >> 4;
      uint32_t it = 0, local_tile = 0;
      bool ok = true;
      for (int tile = tile0; tile < num_tiles && ok; tile += tile_step) {
        const uint32_t acc = local_tile & 1;
        const uint32_t acc_ph = (local_tile >> 1) & 1;
        ++local_tile;
        if (!mbar_wait(&tmem_empty[acc], acc_ph ^ 1, abort_flag)) {
          if (lane == 0) {
            atomicExch(args.status, FSB_ERR_WAIT_TIMEOUT_TMEM_EMPTY);
            *abort_flag = 1;
          }
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % STAGES2;
          const uint32_t ph = (it / STAGES2) & 1;
          if (!mbar_wait(&full_bar[s], ph, abort_flag)) {
            if (lane == 0) {
              atomicExch(args.status, FSB_ERR_WAIT_TIMEOUT_FULL);
              *abort_flag = 1;
            }
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * STAGE2_BYTES);
          const uint64_t da = make_smem_desc_sw128(sa, a_lbo, 1024);
          const uint64_t db = make_smem_desc_sw128(sa + A_STAGE_BYTES, b_lbo, 1024);
          const uint32_t e_own = smem_u32(&empty_bar[s]);
          if (elect_one()) {
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k)
              umma_f16_pair(d_tmem, da + k * a_kstep, db + k * b_kstep, idesc, (kb | k) != 0 ? 1u : 0u);
            // the stage is free in both CTAs once these MMAs have read it
            umma_commit_pair(e_own);
            umma_commit_pair(map_to_cta(e_own, 1));
          }
          __syncwarp();
        }
        if (ok) {
          const uint32_t f_own = smem_u32(&tmem_full[acc]);
          if (elect_one()) {
            umma_commit_pair(f_own);
            umma_commit_pair(map_to_cta(f_own, 1));
          }
          __syncwarp();
        }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5, both CTAs)
    const int quarter = warp & 3;
    uint32_t local_tile = 0;
    for (int tile = tile0; tile < num_tiles; tile += tile_step) {
      int tm2, tn;
      if (args.upper_only) {
        upper_tile_coords(tile, tiles_m, tm2, tn);
      } else {
        tile_coords(tile, tiles_m, tiles_n, tm2, tn);
        if (spread) tm2 = spread_over_row_blocks(tm2, tiles_m, args.d_peer_n);
      }
      const int tm = tm2 * 2 + static_cast<int>(rank);
      const uint32_t acc = local_tile & 1;
      const uint32_t acc_ph = (local_tile >> 1) & 1;
      ++local_tile;
      if (!mbar_wait(&tmem_full[acc], acc_ph, abort_flag)) {
        if (lane == 0) {
          atomicExch(args.status, FSB_ERR_WAIT_TIMEOUT_TMEM_FULL);
          *abort_flag = 1;
        }
        break;
      }
      tc_fence_after();
      store_tile(args, 0, tm, tn, tmem_base + acc * BN + (static_cast<uint32_t>(quarter * 32) << 16),
                 reinterpret_cast<float*>(smem + STAGES2 * STAGE2_BYTES + 256) + (warp - 2) * 32 * 33, quarter, lane);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&tmem_empty[acc]), 0));
    }
  }

  // Common exit: every loop above is bounded, so all warps of both CTAs arrive here. Neither CTA may
  // leave (its barriers and shared memory are targets of the peer) before both are done.
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    if (*abort_flag) {
      const unsigned long long t0 = clock64();
      while (clock64() - t0 < 2000000ull) {
      }
    }
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

int g_num_sms[64] = {0};
int g_pair_clusters[64] = {0};   // co-resident clusters of the two-SM kernel, per device (-1: unusable)

}  // namespace

FsbEncodeTiledFn fsb_get_encode_tiled() {
  static FsbEncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<FsbEncodeTiledFn>(p);
    }
  }
  return fn;
}

int fsb_make_tmap_2d(CUtensorMap* map, const void* base, CUtensorMapDataType dtype, int elem_size,
                     uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows,
                     uint32_t box_cols) {
  FsbEncodeTiledFn enc = fsb_get_encode_tiled();
  if (enc == nullptr) return FSB_ERR_TMA_ENCODE;
  // The driver entry point needs a current context on the calling thread; threads that
  // only ever launched kernels through the runtime (e.g. autograd workers) may not have
  // one bound yet.
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) {
    cudaFree(nullptr);
    ctx_bound = true;
  }
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (ld * elem_size) % 16 != 0)
    return FSB_ERR_BAD_ARG;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * static_cast<uint64_t>(elem_size)};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, dtype, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    fprintf(stderr,
            "[fsb200] cuTensorMapEncodeTiled failed (CUresult %d): base=%p rows=%llu cols=%llu ld=%llu "
            "box=[%u,%u] elem=%d\n",
            static_cast<int>(r), base, static_cast<unsigned long long>(rows),
            static_cast<unsigned long long>(cols), static_cast<unsigned long long>(ld), box_rows,
            box_cols, elem_size);
    return FSB_ERR_TMA_ENCODE;
  }
  return FSB_OK;
}

int fsb_make_tmap_2d_plain(CUtensorMap* map, const void* base, CUtensorMapDataType dtype,
                           int elem_size, uint64_t rows, uint64_t cols, uint64_t ld,
                           uint32_t box_rows, uint32_t box_cols) {
  FsbEncodeTiledFn enc = fsb_get_encode_tiled();
  if (enc == nullptr) return FSB_ERR_TMA_ENCODE;
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) {
    cudaFree(nullptr);
    ctx_bound = true;
  }
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (ld * elem_size) % 16 != 0)
    return FSB_ERR_BAD_ARG;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * static_cast<uint64_t>(elem_size)};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, dtype, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                   CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    fprintf(stderr, "[fsb200] cuTensorMapEncodeTiled (plain) failed (CUresult %d)\n", static_cast<int>(r));
    return FSB_ERR_TMA_ENCODE;
  }
  return FSB_OK;
}

static int g_use_pairs_value();
static inline bool g_use_pairs_fwd() { return g_use_pairs_value() != 0; }

// D[r][c] = D[c][r] for every element of the 256x256 tiles strictly below the diagonal of a square bf16
// matrix: completes a symmetric product of which only the upper tiles were computed. 32x32 tiles through
// shared memory, so both the reads and the writes are contiguous.
__global__ void __launch_bounds__(256)
mirror_upper_kernel(__nv_bfloat16* __restrict__ d, long long ldd, int n) {
  __shared__ __nv_bfloat16 t[32][34];
  const int br = blockIdx.y, bc = blockIdx.x;          // destination block (rows br*32.., columns bc*32..)
  if ((br * 32) / 256 <= (bc * 32) / 256) return;      // only blocks inside the tiles below the diagonal
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  for (int i = ty; i < 32; i += 8) {
    const int r = bc * 32 + i, c = br * 32 + tx;       // source element (the transposed position)
    if (r < n && c < n) t[i][tx] = d[r * ldd + c];
  }
  __syncthreads();
  for (int i = ty; i < 32; i += 8) {
    const int r = br * 32 + i, c = bc * 32 + tx;
    if (r < n && c < n) d[r * ldd + c] = t[tx][i];
  }
}

static int gemm_pair_launch(const void* a, const void* b, void* d, const void* c, int M, int N, int K,
                            long long lda, long long ldb, long long ldd, long long ldc, int a_mn, int b_mn,
                            int d_fp32, int c_fp32, float alpha, float beta, int accumulate,
                            long long d_block_rows, long long d_block_stride, const unsigned long long* d_peer,
                            int d_peer_n, int* status, cudaStream_t stream, int upper_only = 0) {
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return FSB_ERR_BAD_ARG;
  if (g_pair_clusters[dev] == 0) {
    g_pair_clusters[dev] = -1;
    if (cudaFuncSetAttribute(gemm_bf16_2sm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM2_BYTES) ==
        cudaSuccess) {
      cudaLaunchConfig_t cfg{};
      cfg.gridDim = dim3(2, 1, 1);
      cfg.blockDim = dim3(NUM_THREADS, 1, 1);
      cfg.dynamicSmemBytes = SMEM2_BYTES;
      cudaLaunchAttribute at{};
      at.id = cudaLaunchAttributeClusterDimension;
      at.val.clusterDim.x = 2;
      at.val.clusterDim.y = 1;
      at.val.clusterDim.z = 1;
      cfg.attrs = &at;
      cfg.numAttrs = 1;
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, gemm_bf16_2sm_kernel, &cfg) == cudaSuccess && n > 0)
        g_pair_clusters[dev] = n;
    }
    cudaGetLastError();
  }
  if (g_pair_clusters[dev] < 0) return FSB_ERR_TOO_LARGE;
  CUtensorMap map_a, map_b;
  int rc;
  if (!a_mn) rc = fsb_make_tmap_2d(&map_a, a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, K, lda, BM, BK);
  else rc = fsb_make_tmap_2d(&map_a, a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, M, lda, BK, 64);
  if (rc != FSB_OK) return rc;
  if (!b_mn) rc = fsb_make_tmap_2d(&map_b, b, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, K, ldb, BN_HALF, BK);
  else rc = fsb_make_tmap_2d(&map_b, b, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, N, ldb, BK, 64);
  if (rc != FSB_OK) return rc;
  GemmArgs args{};
  args.M = M; args.N = N; args.K = K; args.a_mn = a_mn; args.b_mn = b_mn;
  args.d = d; args.ldd = ldd; args.d_fp32 = d_fp32; args.c = c; args.ldc = ldc; args.c_fp32 = c_fp32;
  args.alpha = alpha; args.beta = beta; args.accumulate = accumulate;
  args.d_peer_remote = d_peer_n > 0;
  if (d_peer_n < 0) d_peer_n = -d_peer_n;
  args.d_block_rows = d_block_rows; args.d_block_stride = d_block_stride; args.d_peer_n = d_peer_n;
  args.status = status;
  for (int i = 0; i < d_peer_n; ++i) args.d_peer[i] = reinterpret_cast<void*>(d_peer[i]);
  long long tiles = static_cast<long long>((M + 2 * BM - 1) / (2 * BM)) * ((N + BN - 1) / BN);
  // a symmetric product into a plain bf16 matrix: the tiles on or above the diagonal, then their mirror image
  upper_only = upper_only && M == N && !d_fp32 && !accumulate && d_peer_n == 0 && d_block_rows == 0 && M > 2 * BM;
  if (upper_only) {
    const long long T = (M + 2 * BM - 1) / (2 * BM);
    tiles = T * (T + 1) / 2;
    args.upper_only = 1;
  }
  const int clusters = tiles < g_pair_clusters[dev] ? static_cast<int>(tiles) : g_pair_clusters[dev];
  gemm_bf16_2sm_kernel<<<2 * clusters, NUM_THREADS, SMEM2_BYTES, stream>>>(map_a, map_b, args);
  if (cudaGetLastError() != cudaSuccess) return FSB_ERR_LAUNCH;
  if (upper_only) {
    const unsigned nb = static_cast<unsigned>((M + 31) / 32);
    mirror_upper_kernel<<<dim3(nb, nb), 256, 0, stream>>>(static_cast<__nv_bfloat16*>(d), ldd, M);
    if (cudaGetLastError() != cudaSuccess) return FSB_ERR_LAUNCH;
  }
  return FSB_OK;
}

// D = alpha * A.B^T + beta * C (+ D). Shapes in elements; see the header comment
// for the meaning of a_mn / b_mn. `status` is a device int the kernel writes an
// error code to when a bounded wait runs out (left untouched otherwise).
FSB_API int fsb_gemm_bf16(const void* a, const void* b, void* d, const void* c, int M, int N, int K,
                          long long lda, long long ldb, long long ldd, long long ldc, int a_mn,
                          int b_mn, int d_fp32, int c_fp32, float alpha, float beta, int accumulate,
                          long long d_block_rows, long long d_block_stride,
                          const unsigned long long* d_peer, int d_peer_n, int* status, int max_ctas,
                          cudaStream_t stream);

// Grouped GEMMs for mixture-of-experts layers (see GemmArgs::group_mode). Row groups start on
// multiples of 128 and are zero-padded to multiples of 128.
//   mode 1: D[R, N] = A[R, K] . B_e[N, K]^T (b_mn = 0, B is [E*N, K]) or A[R, K] . B_e[K, N]
//           (b_mn = 1, B is [E*K, N]); tile_expert[t] names the expert of m-tile t, *num_mtiles the
//           number of valid m-tiles (device memory: no host synchronisation), max_mtiles bounds it.
//   mode 2: D[E, M, N] = sum over each expert's rows of A[r, :M]^T B[r, :N] (A, B row-major
//           [R, M] / [R, N]); group_offs is the int[E+1] array of padded row offsets.
FSB_API int fsb_gemm_bf16_grouped_ex(const void* a, const void* b, void* d, int mode, int num_groups, int M,
                                     int N, int K, long long lda, long long ldb, long long ldd, int b_mn,
                                     int d_fp32, int accumulate, const int* tile_expert,
                                     const int* num_mtiles, const int* group_offs, int max_rows,
                                     const void* c, long long ldc, int c_fp32, float alpha, float beta,
                                     int* status, cudaStream_t stream);

FSB_API int fsb_gemm_bf16_grouped(const void* a, const void* b, void* d, int mode, int num_groups, int M,
                                  int N, int K, long long lda, long long ldb, long long ldd, int b_mn,
                                  int d_fp32, int accumulate, const int* tile_expert,
                                  const int* num_mtiles, const int* group_offs, int max_rows,
                                  int* status, cudaStream_t stream) {
  return fsb_gemm_bf16_grouped_ex(a, b, d, mode, num_groups, M, N, K, lda, ldb, ldd, b_mn, d_fp32, accumulate,
                                  tile_expert, num_mtiles, group_offs, max_rows, nullptr, 0, 0, 1.f, 0.f, status,
                                  stream);
}

// The same with the dense GEMM's epilogue: D = alpha * product + beta * C, where C has D's layout
// ([R, N] rows for mode 1, [E, M, N] for mode 2).
FSB_API int fsb_gemm_bf16_grouped_ex(const void* a, const void* b, void* d, int mode, int num_groups, int M,
                                     int N, int K, long long lda, long long ldb, long long ldd, int b_mn,
                                     int d_fp32, int accumulate, const int* tile_expert,
                                     const int* num_mtiles, const int* group_offs, int max_rows,
                                     const void* c, long long ldc, int c_fp32, float alpha, float beta,
                                     int* status, cudaStream_t stream) {
  if (mode != 1 && mode != 2) return FSB_ERR_BAD_ARG;
  CUtensorMap map_a, map_b;
  int rc;
  GemmArgs args{};
  if (mode == 1) {
    // A [max_rows, K] K-major; B stacked over experts
    rc = fsb_make_tmap_2d(&map_a, a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, max_rows, K, lda, BM, BK);
    if (rc != FSB_OK) return rc;
    if (!b_mn) rc = fsb_make_tmap_2d(&map_b, b, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                                     static_cast<uint64_t>(num_groups) * N, K, ldb, BN, BK);
    else rc = fsb_make_tmap_2d(&map_b, b, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                               static_cast<uint64_t>(num_groups) * K, N, ldb, BK, 64);
    if (rc != FSB_OK) return rc;
    args.M = max_rows; args.N = N; args.K = K; args.a_mn = 0; args.b_mn = b_mn;
    args.b_group_rows = b_mn ? K : N;
  } else {
    // A [max_rows, M], B [max_rows, N] both MN-major; contraction over the rows of each group
    rc = fsb_make_tmap_2d(&map_a, a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, max_rows, M, lda, BK, 64);
    if (rc != FSB_OK) return rc;
    rc = fsb_make_tmap_2d(&map_b, b, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, max_rows, N, ldb, BK, 64);
    if (rc != FSB_OK) return rc;
    args.M = M; args.N = N; args.K = max_rows; args.a_mn = 1; args.b_mn = 1;
  }
  args.d = d; args.ldd = ldd; args.d_fp32 = d_fp32; args.alpha = alpha; args.beta = c != nullptr ? beta : 0.f;
  args.c = c; args.ldc = ldc; args.c_fp32 = c_fp32;
  args.accumulate = accumulate; args.group_mode = mode; args.num_groups = num_groups;
  args.tile_expert = tile_expert; args.num_mtiles = num_mtiles; args.group_offs = group_offs;
  args.status = status;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return FSB_ERR_BAD_ARG;
  static bool attr_set[64] = {false};
  if (!attr_set[dev]) {
    if (cudaFuncSetAttribute(gemm_bf16_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             SMEM_BYTES) != cudaSuccess)
      return FSB_ERR_LAUNCH;
    attr_set[dev] = true;
  }
  if (g_num_sms[dev] == 0) cudaDeviceGetAttribute(&g_num_sms[dev], cudaDevAttrMultiProcessorCount, dev);
  const long long tiles = static_cast<long long>((args.M + BM - 1) / BM) * ((N + BN - 1) / BN) *
                          (mode == 2 ? num_groups : 1);
  const int grid = tiles < g_num_sms[dev] ? static_cast<int>(tiles) : g_num_sms[dev];
  AgArgs none{};
  gemm_bf16_kernel<false><<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(map_a, map_b, args, none);
  return cudaGetLastError() == cudaSuccess ? FSB_OK : FSB_ERR_LAUNCH;
}

FSB_API int fsb_gemm_bf16(const void* a, const void* b, void* d, const void* c, int M, int N, int K,
                          long long lda, long long ldb, long long ldd, long long ldc, int a_mn,
                          int b_mn, int d_fp32, int c_fp32, float alpha, float beta, int accumulate,
                          long long d_block_rows, long long d_block_stride,
                          const unsigned long long* d_peer, int d_peer_n, int* status, int max_ctas,
                          cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return FSB_ERR_BAD_ARG;
  // bit 1 of `accumulate`: the product is symmetric (A B^T with B = A, or a symmetric A times itself) and only
  // its upper tiles need computing; honoured by the two-SM kernel for square bf16 outputs, ignored otherwise
  const int upper_only = (accumulate >> 1) & 1;
  accumulate &= 1;
  // a negative block count means: the blocks are in this GPU's own memory (no row-segment staging)
  const int d_peer_remote = d_peer_n > 0;
  if (d_peer_n < 0) d_peer_n = -d_peer_n;
  if (d_peer_n > 16 || (d_peer_n > 0 && d_block_rows <= 0)) return FSB_ERR_BAD_ARG;
  if (g_use_pairs_fwd() && M >= 2 * BM && N >= BN && max_ctas <= 0) {
    const int rc2 = gemm_pair_launch(a, b, d, c, M, N, K, lda, ldb, ldd, ldc, a_mn, b_mn, d_fp32, c_fp32, alpha,
                                     beta, accumulate, d_block_rows, d_block_stride, d_peer,
                                     d_peer_remote ? d_peer_n : -d_peer_n, status, stream, upper_only);
    if (rc2 != FSB_ERR_TOO_LARGE) return rc2;   // TOO_LARGE here means "pairs unusable on this device"
  }
  CUtensorMap map_a, map_b;
  int rc;
  if (!a_mn) {
    rc = fsb_make_tmap_2d(&map_a, a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, K, lda, BM, BK);
  } else {
    rc = fsb_make_tmap_2d(&map_a, a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, M, lda, BK, 64);
  }
  if (rc != FSB_OK) return rc;
  if (!b_mn) {
    rc = fsb_make_tmap_2d(&map_b, b, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, K, ldb, BN, BK);
  } else {
    rc = fsb_make_tmap_2d(&map_b, b, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, N, ldb, BK, 64);
  }
  if (rc != FSB_OK) return rc;

  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return FSB_ERR_BAD_ARG;
  static bool plain_attr_set[64] = {false};
  if (!plain_attr_set[dev]) {
    if (cudaFuncSetAttribute(gemm_bf16_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             SMEM_BYTES) != cudaSuccess)
      return FSB_ERR_LAUNCH;
    plain_attr_set[dev] = true;
  }
  if (g_num_sms[dev] == 0) cudaDeviceGetAttribute(&g_num_sms[dev], cudaDevAttrMultiProcessorCount, dev);
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  int grid = tiles < g_num_sms[dev] ? tiles : g_num_sms[dev];
  if (max_ctas > 0 && grid > max_ctas) grid = max_ctas;
  GemmArgs args{};
  args.M = M; args.N = N; args.K = K; args.a_mn = a_mn; args.b_mn = b_mn;
  args.d = d; args.ldd = ldd; args.d_fp32 = d_fp32; args.c = c; args.ldc = ldc; args.c_fp32 = c_fp32;
  args.alpha = alpha; args.beta = beta; args.accumulate = accumulate;
  args.d_block_rows = d_block_rows; args.d_block_stride = d_block_stride; args.d_peer_n = d_peer_n;
  args.d_peer_remote = d_peer_remote;
  args.status = status;
  for (int i = 0; i < d_peer_n; ++i) args.d_peer[i] = reinterpret_cast<void*>(d_peer[i]);
  AgArgs none{};
  gemm_bf16_kernel<false><<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(map_a, map_b, args, none);
  return cudaGetLastError() == cudaSuccess ? FSB_OK : FSB_ERR_LAUNCH;
}

// 0: one-SM kernel only; 1 (default): dense GEMMs with M >= 256 and N >= 256 run on SM pairs.
static int g_use_pairs = 1;
static int g_use_pairs_value() { return g_use_pairs; }
FSB_API int fsb_gemm_set_pair_mode(int on) {
  g_use_pairs = on;
  return FSB_OK;
}

// All-gather -> GEMM in one kernel: D[M,N] = A[M,K] . W[N,K]^T where W is row-sharded over
// `world` ranks (peer_shards[r] = address of rank r's rows, shard_rows each; the last rank may
// hold padding). `gathered` receives the full weight (it is the GEMM's B operand and stays valid
// afterwards, e.g. for the backward pass). `counters` is a zero-initialised int array of
// ceil(N/256) entries that belongs to this weight; `call_index` counts calls using it (1, 2, ...).
// `peer_flags` / `epoch`: this rank's flag row saying from which epoch on the peers' shards are
// valid (null: no wait). Launched cooperatively so that stager and GEMM CTAs are co-resident.
FSB_API int fsb_gemm_bf16_allgather(const void* a, const unsigned long long* peer_shards, void* gathered,
                                    void* d, int M, int N, int K, long long lda, long long ldd,
                                    int d_fp32, int world, int shard_rows, int* counters, int call_index,
                                    int n_stagers, const void* peer_flags, unsigned epoch,
                                    unsigned max_polls, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0 || world < 1 || world > AG_MAX_RANKS) return FSB_ERR_BAD_ARG;
  const long long shard_bytes = static_cast<long long>(shard_rows) * K * 2;
  if (shard_bytes % AG_PIECE != 0 || (static_cast<long long>(BN) * K * 2) % AG_PIECE != 0)
    return FSB_ERR_BAD_ARG;
  CUtensorMap map_a, map_b;
  int rc = fsb_make_tmap_2d(&map_a, a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, K, lda, BM, BK);
  if (rc != FSB_OK) return rc;
  rc = fsb_make_tmap_2d(&map_b, gathered, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, K, K, BN, BK);
  if (rc != FSB_OK) return rc;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return FSB_ERR_BAD_ARG;
  static bool attr_set[64] = {false};
  if (!attr_set[dev]) {
    if (cudaFuncSetAttribute(gemm_bf16_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             SMEM_BYTES) != cudaSuccess)
      return FSB_ERR_LAUNCH;
    attr_set[dev] = true;
  }
  if (g_num_sms[dev] == 0) cudaDeviceGetAttribute(&g_num_sms[dev], cudaDevAttrMultiProcessorCount, dev);
  if (n_stagers < 1) n_stagers = 1;
  if (n_stagers > g_num_sms[dev] / 2) n_stagers = g_num_sms[dev] / 2;
  GemmArgs args{};
  args.M = M; args.N = N; args.K = K; args.d = d; args.ldd = ldd; args.d_fp32 = d_fp32;
  args.alpha = 1.f; args.status = status;
  AgArgs ag{};
  for (int r = 0; r < world; ++r) ag.peer[r] = reinterpret_cast<const uint8_t*>(peer_shards[r]);
  ag.local = static_cast<uint8_t*>(gathered);
  ag.shard_bytes = shard_bytes;
  ag.total_bytes = static_cast<long long>(N) * K * 2;
  ag.chunk_bytes = static_cast<long long>(BN) * K * 2;
  ag.counters = counters;
  ag.call_index = call_index;
  ag.n_stagers = n_stagers;
  ag.peer_flags = static_cast<const uint32_t*>(peer_flags);
  ag.world = peer_flags ? world : 0;
  ag.epoch = epoch;
  ag.max_polls = max_polls;
  const int grid = g_num_sms[dev];
  void* params[] = {&map_a, &map_b, &args, &ag};
  cudaError_t e = cudaLaunchCooperativeKernel(reinterpret_cast<void*>(gemm_bf16_kernel<true>), dim3(grid),
                                              dim3(NUM_THREADS), params, SMEM_BYTES, stream);
  return e == cudaSuccess ? FSB_OK : FSB_ERR_LAUNCH;
}
