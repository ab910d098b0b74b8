// Causal flash-attention backward for sm_100a (head_dim 128, GQA), bf16.
//
// One CTA owns a 128-row key/value tile of one KV head and walks every (query tile of 64 rows at or
// below the diagonal, query head of the group) pair, in the order TileWalk defines (by default from the
// last query tile down, the heads of the group inside).
// Everything is computed transposed so that the kv index is the MMA M dimension
// (= TMEM lane = softmax thread) and no operand needs a transpose copy:
//   S^T  = K Q^T          A = K  (K-major)      B = Q  (K-major)        -> TMEM S   (64 columns)
//   dP^T = V dO^T         A = V  (K-major)      B = dO (K-major)        -> TMEM dP  (64 columns)
//   P^T  = exp2(S^T*c - lse),  dS^T = P^T (dP^T - delta)   compute warps -> bf16 smem (two buffers each)
//   dV  += P^T  dO        A = P^T  (K-major)    B = dO (same tile, MN-major)
//   dK  += dS^T Q         A = dS^T (K-major)    B = Q  (same tile, MN-major)
//   dQ^T = K^T dS         A = K (MN-major)      B = dS^T (same tile, MN-major) -> TMEM dQ[it & 1] (64 columns)
// The softmax scale of dS is applied where the products leave the chip (dQ drain, dK epilogue).
//
// Warp roles (448 threads): warp 0 TMA producer (K, V once; Q/dO tiles through a 3-stage ring),
// warp 1 MMA issuer (the whole warp walks the loop, one elected lane issues), warps 2..9 compute
// (two per TMEM lane quarter, 32 query columns each), warps 10..13 dQ drain: dQ^T goes TMEM ->
// registers -> red.global.add.f32 into a fp32 [B*S, Hq*128] accumulator; a warp's 32 lanes are 32
// consecutive d, so every reduction instruction covers one 128-byte line (measured: the same
// 25 B/clk/SM as a bulk tensor reduce-add, without the shared-memory staging pass).
//
// Schedule. The compute warps of tile i read S(i), dP(i) into registers and release the two TMEM
// buffers at once; the MMA warp then issues S(i+1), dP(i+1) (they run while tile i is being
// exponentiated), and dV(i), dK(i), dQ(i) as soon as P^T(i), dS^T(i) are stored. The tensor pipe
// executes in issue order, so "S(i), dP(i) complete" also means "every product of tile i-2 is
// complete": that one wait also frees the P^T / dS^T buffers of tile i-2 for tile i.
// TMEM: S (64 columns) + dP (64) + dQ[2] (128) + dV (128) + dK (128) = 512 columns.
//
// Ordered mode (BwdArgs::turns != nullptr): the sum that forms dQ gets a fixed order, so two runs give
// the same bits. Every (batch, query head, query tile) has a turn counter; the CTA of kv tile t adds its
// contribution only when the counter shows that kv tiles 0..t-1 have added theirs (4 drain warps each, so
// it waits for 4 t), and raises it afterwards (fence, then one atomic per drain warp). CTAs take their
// (head, kv tile) from a ticket counter instead of blockIdx, in the same longest-first order: a CTA that
// holds ticket n knows that every ticket below n is held by a CTA that is already running, and the CTA a
// turn waits for always has a lower ticket, so the waits cannot deadlock whatever order the hardware
// starts blocks in. The waits are bounded like every other wait of the kernel.
#include "common.cuh"

namespace {
using namespace fsb;

constexpr int HD = 128;
constexpr int BKV = 128;
constexpr int BQ = 64;
constexpr int QSTAGES = 3;
constexpr int KV_TILE_BYTES = BKV * HD * 2;  // 32 KB, two chunks of 16 KB
constexpr int Q_TILE_BYTES = BQ * HD * 2;    // 16 KB, two chunks of 8 KB
constexpr int PT_BYTES = BKV * BQ * 2;       // 16 KB
constexpr int STATS_BYTES = 8 * 64 * 4;      // per compute warp: [32 lse | 32 delta]
constexpr int SMEM_BWD = 2 * KV_TILE_BYTES + 2 * QSTAGES * Q_TILE_BYTES + 4 * PT_BYTES + STATS_BYTES + 256;
static_assert(SMEM_BWD <= 232448, "shared memory budget");
constexpr int THREADS = 448;

struct BwdArgs {
  int S, Hq, Hkv;
  float scale_log2, scale;
  const float* lse;    // [B, Hq, S]
  const float* delta;  // [B, Hq, S]
  float* dq_acc;       // [B*S, Hq*128] fp32, zero-initialised
  int heads_inner;     // walk order of the (query tile, head) pairs, see TileWalk
  int* turns;          // ordered mode: [B*Hq*(S/64)] turn counters followed by one ticket counter, all zero; else null
  __nv_bfloat16* dk;
  long long lddk;
  __nv_bfloat16* dv;
  long long lddv;
  int* status;
};

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void red_add_f32(float* p, float v) {
  asm volatile("red.global.add.f32 [%0], %1;" ::"l"(p), "f"(v) : "memory");
}

// The order in which a CTA visits its (query tile, head of the group) pairs.
//   heads_inner == 0: head by head, query tiles ascending from the diagonal.
//   heads_inner == 1: query tiles descending from the last one, the heads of the group inside. Every CTA of
//     a kv head then starts on the same tile and a CTA with a later kv tile simply stops earlier, so in the
//     ordered mode a CTA runs one hand-over behind its predecessor from the first tile to the last and
//     never has to catch up with it again (head by head it would wait at every change of head).
struct TileWalk {
  int qt, g;
  __device__ __forceinline__ TileWalk(int first, int n_qt, int heads_inner)
      : qt(heads_inner ? first + n_qt - 1 : first), g(0) {}
  __device__ __forceinline__ void next(int first, int n_qt, int G, int heads_inner) {
    if (heads_inner) {
      if (++g == G) {
        g = 0;
        --qt;
      }
    } else if (++qt == first + n_qt) {
      qt = first;
      ++g;
    }
  }
};

// Lane 0 of a drain warp waits until `*ctr` reaches `want` (acquire), bounded.
constexpr uint32_t kTurnSpin = 1u << 21;
__device__ __forceinline__ bool turn_wait(const int* ctr, int want, volatile int* abort_flag,
                                          const volatile int* status) {
#pragma unroll 1
  for (uint32_t i = 0; i < kTurnSpin; ++i) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(ctr) : "memory");
    if (v >= want) return true;
    if (i > 16) __nanosleep(200);
    if ((i & 63) == 63 && *abort_flag) return false;
    if ((i & 1023) == 1023 && *status != 0) return false;   // another CTA gave up: do not wait out the limit
  }
  return false;
}

__global__ void __launch_bounds__(THREADS, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do,
                const BwdArgs args) {
  extern __shared__ __align__(1024) uint8_t smem[];   // no slack: the budget is used to the last KB
  uint8_t* sK = smem;
  uint8_t* sV = sK + KV_TILE_BYTES;
  uint8_t* sQ = sV + KV_TILE_BYTES;                  // [QSTAGES][Q_TILE_BYTES]
  uint8_t* sDO = sQ + QSTAGES * Q_TILE_BYTES;        // [QSTAGES][Q_TILE_BYTES]
  uint8_t* sPT = sDO + QSTAGES * Q_TILE_BYTES;       // P^T [2]
  uint8_t* sDST = sPT + 2 * PT_BYTES;                // dS^T [2]
  float* s_stats = reinterpret_cast<float*>(sDST + 2 * PT_BYTES);
  uint64_t* bars = reinterpret_cast<uint64_t*>(sDST + 2 * PT_BYTES + STATS_BYTES);
  uint64_t* kv_full = bars;          // 1
  uint64_t* qdo_full = bars + 1;     // [3]
  uint64_t* qdo_empty = bars + 4;    // [3]
  uint64_t* sdp_full = bars + 7;     // S^T and dP^T of a tile are in TMEM
  uint64_t* sdp_free = bars + 8;     // compute warps have read them out
  uint64_t* pds_full = bars + 9;     // compute warps stored P^T and dS^T
  uint64_t* dq_full = bars + 10;     // [2]
  uint64_t* dq_free = bars + 12;     // [2] drain warps have read dQ^T out of TMEM
  uint64_t* all_done = bars + 14;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 20);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* ticket_slot = reinterpret_cast<int*>(tmem_slot + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // x = (kv head, batch) so that CTAs are handed out tile by tile: kv tile 0 has the most
  // query tiles below the diagonal, so ascending y is longest-job-first.
  int work = blockIdx.y * gridDim.x + blockIdx.x;
  if (args.turns != nullptr) {   // ordered mode: the same order, but taken from a ticket counter
    if (threadIdx.x == 0)
      *ticket_slot = atomicAdd(args.turns + static_cast<long long>(args.Hq) * (args.S / BQ) * (gridDim.x / args.Hkv), 1);
    __syncthreads();
    work = *ticket_slot;
  }
  const int kv_tile = work / static_cast<int>(gridDim.x);
  const int bx = work % static_cast<int>(gridDim.x);
  const int hk = bx % args.Hkv, b = bx / args.Hkv;
  const int G = args.Hq / args.Hkv;
  const int kv0 = kv_tile * BKV;
  const int row_base = b * args.S;
  const int qt_first = kv0 / BQ;
  const int n_qt = args.S / BQ - qt_first;   // query tiles per head
  const int n_it = n_qt * G;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int i = 0; i < QSTAGES; ++i) {
      mbar_init(&qdo_full[i], 1);
      mbar_init(&qdo_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&dq_full[i], 1);
      mbar_init(&dq_free[i], 4);
    }
    mbar_init(sdp_full, 1);
    mbar_init(sdp_free, 8);
    mbar_init(pds_full, 8);
    mbar_init(all_done, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if ((smem_u32(smem) & 1023u) != 0) {   // swizzled tiles need 1 KB alignment; uniform for the CTA
    if (threadIdx.x == 0) atomicExch(args.status, FSB_ERR_BAD_ARG);
    return;
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_s = tmem_base;          // 64 columns
  const uint32_t tmem_dp = tmem_base + 64;
  const uint32_t tmem_dq = tmem_base + 128;   // [2] x 64 columns
  const uint32_t tmem_dv = tmem_base + 256;
  const uint32_t tmem_dk = tmem_base + 384;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&map_q);
      tma_prefetch_desc(&map_do);
      mbar_expect_tx(kv_full, 2 * KV_TILE_BYTES);
      tma_load_2d(sK, &map_k, kv_full, hk * HD, row_base + kv0);
      tma_load_2d(sK + KV_TILE_BYTES / 2, &map_k, kv_full, hk * HD + 64, row_base + kv0);
      tma_load_2d(sV, &map_v, kv_full, hk * HD, row_base + kv0);
      tma_load_2d(sV + KV_TILE_BYTES / 2, &map_v, kv_full, hk * HD + 64, row_base + kv0);
      int st = 0;
      uint32_t ph = 0;
      TileWalk walk(qt_first, n_qt, args.heads_inner);
      for (int it = 0; it < n_it; ++it) {
        const int h = hk * G + walk.g;
        const int qt = walk.qt;
        walk.next(qt_first, n_qt, G, args.heads_inner);
        if (!mbar_wait(&qdo_empty[st], ph ^ 1, abort_flag)) {
          atomicExch(args.status, FSB_ERR_WAIT_TIMEOUT_EMPTY);
          *abort_flag = 1;
          break;
        }
        mbar_expect_tx(&qdo_full[st], 2 * Q_TILE_BYTES);
        uint8_t* q = sQ + st * Q_TILE_BYTES;
        uint8_t* d = sDO + st * Q_TILE_BYTES;
        const int row = row_base + qt * BQ;
        tma_load_2d(q, &map_q, &qdo_full[st], h * HD, row);
        tma_load_2d(q + Q_TILE_BYTES / 2, &map_q, &qdo_full[st], h * HD + 64, row);
        tma_load_2d(d, &map_do, &qdo_full[st], h * HD, row);
        tma_load_2d(d + Q_TILE_BYTES / 2, &map_do, &qdo_full[st], h * HD + 64, row);
        if (++st == QSTAGES) {
          st = 0;
          ph ^= 1;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    // The whole warp walks the loop (waits, descriptor arithmetic: warp-uniform); one elected lane
    // issues the tcgen05 instructions.
    {
      const uint32_t idesc_sdp = make_idesc(BKV, BQ, 1, 1, 0, 0);   // M=128 kv, N=64 q
      const uint32_t idesc_dkv = make_idesc(BKV, HD, 1, 1, 0, 1);   // M=128 kv, N=128 d, B MN-major
      const uint32_t idesc_dq = make_idesc(HD, BQ, 1, 1, 1, 1);     // M=128 d,  N=64 q, both MN-major
      // descriptors of the tile bases; a step inside a tile adds (bytes >> 4) to the address field
      const uint64_t dk_k = make_smem_desc_sw128(smem_u32(sK), 16, 1024);                    // K, K-major
      const uint64_t dv_k = make_smem_desc_sw128(smem_u32(sV), 16, 1024);                    // V, K-major
      const uint64_t dk_mn = make_smem_desc_sw128(smem_u32(sK), KV_TILE_BYTES / 2, 1024);    // K, MN-major
      bool ok = mbar_wait(kv_full, 0, abort_flag);

      auto wait_q = [&](int it) -> bool {
        return mbar_wait(&qdo_full[it % QSTAGES], (it / QSTAGES) & 1, abort_flag);
      };
      // S^T(it) = K Q^T and dP^T(it) = V dO^T
      auto issue_sdp = [&](int it) {
        const uint64_t dq_k = make_smem_desc_sw128(smem_u32(sQ + (it % QSTAGES) * Q_TILE_BYTES), 16, 1024);
        const uint64_t ddo_k = make_smem_desc_sw128(smem_u32(sDO + (it % QSTAGES) * Q_TILE_BYTES), 16, 1024);
        if (elect_one()) {
          {
#pragma unroll
            for (int k = 0; k < HD / 16; ++k) {
              const uint32_t ko = ((k >> 2) * (KV_TILE_BYTES / 2) + (k & 3) * 32) >> 4;
              const uint32_t qo = ((k >> 2) * (Q_TILE_BYTES / 2) + (k & 3) * 32) >> 4;
              umma_f16(tmem_s, dk_k + ko, dq_k + qo, idesc_sdp, k != 0);
            }
#pragma unroll
            for (int k = 0; k < HD / 16; ++k) {
              const uint32_t vo = ((k >> 2) * (KV_TILE_BYTES / 2) + (k & 3) * 32) >> 4;
              const uint32_t dof = ((k >> 2) * (Q_TILE_BYTES / 2) + (k & 3) * 32) >> 4;
              umma_f16(tmem_dp, dv_k + vo, ddo_k + dof, idesc_sdp, k != 0);
            }
          }
          umma_commit(sdp_full);
        }
        __syncwarp();
      };

      if (ok && n_it > 0) {
        ok = wait_q(0);
        if (ok) {
          tc_fence_after();
          issue_sdp(0);
        }
      }
      for (int it = 0; it < n_it && ok; ++it) {
        // S(it+1), dP(it+1) as soon as the compute warps have read S(it), dP(it) out of TMEM
        if (it + 1 < n_it) {
          if (!wait_q(it + 1) || !mbar_wait(sdp_free, it & 1, abort_flag)) { ok = false; break; }
          tc_fence_after();
          issue_sdp(it + 1);
        }
        // B operands read MN-major out of the Q / dO tiles: d chunks 8 KB apart (LBO), 8-query
        // groups 1 KB apart (SBO), 16 queries = 2 KB
        const uint64_t dq_mn = make_smem_desc_sw128(smem_u32(sQ + (it % QSTAGES) * Q_TILE_BYTES), Q_TILE_BYTES / 2, 1024);
        const uint64_t ddo_mn = make_smem_desc_sw128(smem_u32(sDO + (it % QSTAGES) * Q_TILE_BYTES), Q_TILE_BYTES / 2, 1024);
        const uint64_t dpt = make_smem_desc_sw128(smem_u32(sPT + (it & 1) * PT_BYTES), 16, 1024);
        const uint64_t dds_k = make_smem_desc_sw128(smem_u32(sDST + (it & 1) * PT_BYTES), 16, 1024);
        const uint64_t dds_mn = make_smem_desc_sw128(smem_u32(sDST + (it & 1) * PT_BYTES), PT_BYTES, 1024);
        // dV += P^T dO ; dK += dS^T Q   (K = 64 queries, 4 steps each)
        if (!mbar_wait(pds_full, it & 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        if (elect_one()) {
          {
#pragma unroll
            for (int k = 0; k < BQ / 16; ++k)
              umma_f16(tmem_dv, dpt + ((k * 32) >> 4), ddo_mn + ((k * 2048) >> 4), idesc_dkv, (it | k) != 0);
#pragma unroll
            for (int k = 0; k < BQ / 16; ++k)
              umma_f16(tmem_dk, dds_k + ((k * 32) >> 4), dq_mn + ((k * 2048) >> 4), idesc_dkv, (it | k) != 0);
          }
          umma_commit(&qdo_empty[it % QSTAGES]);
        }
        __syncwarp();
        if (it > 1) {
          if (!mbar_wait(&dq_free[it & 1], ((it >> 1) - 1) & 1, abort_flag)) { ok = false; break; }
          tc_fence_after();
        }
        // dQ^T = K^T dS: A = K read MN-major (d chunks 16 KB apart, 8-kv groups 1 KB apart), B = dS^T
        // read MN-major (a single 64-query group), K = 128 kv in 8 steps of 2 KB.
        if (elect_one()) {
#pragma unroll
          for (int k = 0; k < BKV / 16; ++k)
            umma_f16(tmem_dq + (it & 1) * 64, dk_mn + ((k * 2048) >> 4), dds_mn + ((k * 2048) >> 4), idesc_dq, k != 0);
          umma_commit(&dq_full[it & 1]);
        }
        __syncwarp();
      }
      if (ok) {
        if (elect_one()) umma_commit(all_done);
        __syncwarp();
      } else if (lane == 0) {
        atomicExch(args.status, FSB_ERR_WAIT_TIMEOUT_FULL);
        *abort_flag = 1;
      }
    }
  } else if (warp < 10) {
    // ------------------------------------------------------------ compute warps
    // Two warps share each TMEM lane quarter and split the 64 query columns between them: every
    // element of the backward pass is independent (no row reductions), so the split needs no exchange.
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;    // 0: query columns [0,32), 1: [32,64)
    const int c0 = half * 32;
    const int r = quarter * 32 + lane;   // kv row inside the tile
    const int kv_row = kv0 + r;
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    const float LOG2E = 1.4426950408889634f;
    bool ok = true;
    float* s_lse = s_stats + (warp - 2) * 64;   // [32 lse | 32 delta] of this warp's 32 queries
    float* s_delta = s_lse + 32;
    // (head, query tile) of the running tile, advanced without divisions
    TileWalk walk(qt_first, n_qt, args.heads_inner);
    // index of this lane's statistic in lse / delta for (head 0 of the group, query 0); B * Hq * S < 2^31 (checked by the host)
    const int stat_base = (b * args.Hq + hk * G) * args.S + c0 + lane;
    float nl = 0.f, nd = 0.f;
    if (n_it > 0) {
      nl = args.lse[stat_base + walk.g * args.S + walk.qt * BQ];
      nd = args.delta[stat_base + walk.g * args.S + walk.qt * BQ];
    }

    for (int it = 0; it < n_it; ++it) {
      const int q0 = walk.qt * BQ;
      __syncwarp();   // the previous tile's reads of the statistics are done
      s_lse[lane] = nl * LOG2E;
      s_delta[lane] = nd;
      __syncwarp();
      walk.next(qt_first, n_qt, G, args.heads_inner);
      if (it + 1 < n_it) {   // next tile's statistics: the loads land while this tile is computed
        nl = args.lse[stat_base + walk.g * args.S + walk.qt * BQ];
        nd = args.delta[stat_base + walk.g * args.S + walk.qt * BQ];
      }
      // S(it), dP(it) complete also says that every product of tile it-2 is complete (one in-order
      // pipe), so P^T[it & 1] and dS^T[it & 1] may be overwritten.
      if (!mbar_wait_warp(sdp_full, it & 1, abort_flag)) { ok = false; break; }
      tc_fence_after();
      uint32_t pk[16], dk[16];
      {
        uint32_t sv[32], dp[32];
        tmem_ld_32x32(tmem_s + lane_off + c0, sv);
        tmem_ld_32x32(tmem_dp + lane_off + c0, dp);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(sdp_free);
        const bool diag = q0 + c0 < kv0 + BKV;   // some (kv, q) pairs of this warp's part are above the diagonal
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const float4 l4 = *reinterpret_cast<const float4*>(s_lse + u * 4);
          const float4 d4 = *reinterpret_cast<const float4*>(s_delta + u * 4);
          float p0 = fast_exp2(fmaf(__uint_as_float(sv[u * 4 + 0]), args.scale_log2, -l4.x));
          float p1 = fast_exp2(fmaf(__uint_as_float(sv[u * 4 + 1]), args.scale_log2, -l4.y));
          float p2 = fast_exp2(fmaf(__uint_as_float(sv[u * 4 + 2]), args.scale_log2, -l4.z));
          float p3 = fast_exp2(fmaf(__uint_as_float(sv[u * 4 + 3]), args.scale_log2, -l4.w));
          if (diag) {
            const int qi = q0 + c0 + u * 4;
            if (kv_row > qi + 0) p0 = 0.f;
            if (kv_row > qi + 1) p1 = 0.f;
            if (kv_row > qi + 2) p2 = 0.f;
            if (kv_row > qi + 3) p3 = 0.f;
          }
          pk[u * 2 + 0] = pack_bf16x2(p0, p1);
          pk[u * 2 + 1] = pack_bf16x2(p2, p3);
          dk[u * 2 + 0] = pack_bf16x2(p0 * (__uint_as_float(dp[u * 4 + 0]) - d4.x),
                                      p1 * (__uint_as_float(dp[u * 4 + 1]) - d4.y));
          dk[u * 2 + 1] = pack_bf16x2(p2 * (__uint_as_float(dp[u * 4 + 2]) - d4.z),
                                      p3 * (__uint_as_float(dp[u * 4 + 3]) - d4.w));
        }
      }
      uint8_t* prow = sPT + (it & 1) * PT_BYTES + r * 128;
      uint8_t* drow = sDST + (it & 1) * PT_BYTES + r * 128;
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int unit = ((c0 >> 3) + u) ^ (r & 7);
        *reinterpret_cast<uint4*>(prow + (unit << 4)) = make_uint4(pk[u * 4], pk[u * 4 + 1], pk[u * 4 + 2], pk[u * 4 + 3]);
        *reinterpret_cast<uint4*>(drow + (unit << 4)) = make_uint4(dk[u * 4], dk[u * 4 + 1], dk[u * 4 + 2], dk[u * 4 + 3]);
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(pds_full);
    }
    if (ok && mbar_wait_warp(all_done, 0, abort_flag)) {
      tc_fence_after();
      __nv_bfloat16* dkrow = args.dk + static_cast<long long>(row_base + kv_row) * args.lddk + hk * HD;
      __nv_bfloat16* dvrow = args.dv + static_cast<long long>(row_base + kv_row) * args.lddv + hk * HD;
      const float sc = args.scale;
#pragma unroll 1
      for (int cc = half * 64; cc < half * 64 + 64; cc += 32) {
        uint32_t a[32], c[32];
        tmem_ld_32x32(tmem_dk + lane_off + cc, a);
        tmem_ld_32x32(tmem_dv + lane_off + cc, c);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; i += 8) {
          uint4 x, y;
          x.x = pack_bf16x2(__uint_as_float(a[i]) * sc, __uint_as_float(a[i + 1]) * sc);
          x.y = pack_bf16x2(__uint_as_float(a[i + 2]) * sc, __uint_as_float(a[i + 3]) * sc);
          x.z = pack_bf16x2(__uint_as_float(a[i + 4]) * sc, __uint_as_float(a[i + 5]) * sc);
          x.w = pack_bf16x2(__uint_as_float(a[i + 6]) * sc, __uint_as_float(a[i + 7]) * sc);
          y.x = pack_bf16x2(__uint_as_float(c[i]), __uint_as_float(c[i + 1]));
          y.y = pack_bf16x2(__uint_as_float(c[i + 2]), __uint_as_float(c[i + 3]));
          y.z = pack_bf16x2(__uint_as_float(c[i + 4]), __uint_as_float(c[i + 5]));
          y.w = pack_bf16x2(__uint_as_float(c[i + 6]), __uint_as_float(c[i + 7]));
          *reinterpret_cast<uint4*>(dkrow + cc + i) = x;
          *reinterpret_cast<uint4*>(dvrow + cc + i) = y;
        }
      }
    } else if (lane == 0) {
      atomicExch(args.status, FSB_ERR_WAIT_TIMEOUT_TMEM_FULL);
      *abort_flag = 1;
    }
  } else {
    // ------------------------------------------------------------ dQ drain warps
    const int quarter = warp & 3;
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    const int d = quarter * 32 + lane;   // dQ^T lane = head-dim index
    const float sc = args.scale;
    const long long ldq = static_cast<long long>(args.Hq) * HD;
    TileWalk walk(qt_first, n_qt, args.heads_inner);
    int* prev_turn = nullptr;
    for (int it = 0; it < n_it; ++it) {
      if (!mbar_wait_warp(&dq_full[it & 1], (it >> 1) & 1, abort_flag)) {
        if (lane == 0) {
          atomicExch(args.status, FSB_ERR_WAIT_TIMEOUT_TMEM_FULL);
          *abort_flag = 1;
        }
        break;
      }
      tc_fence_after();
      uint32_t v0[32], v1[32];
      tmem_ld_32x32(tmem_dq + lane_off + (it & 1) * 64, v0);
      tmem_ld_32x32(tmem_dq + lane_off + (it & 1) * 64 + 32, v1);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&dq_free[it & 1]);
      int* turn = nullptr;
      if (args.turns != nullptr) {
        // Raise the previous tile's turn first: its additions were issued an iteration ago and have mostly
        // been performed, so the fence that orders them before the counter costs little here, while a fence
        // right behind the additions would wait for all of them.
        if (prev_turn != nullptr) {
          __syncwarp();
          if (lane == 0) {
            __threadfence();
            atomicAdd(prev_turn, 1);
          }
        }
        turn = args.turns + (static_cast<long long>(b) * args.Hq + hk * G + walk.g) * (args.S / BQ) + walk.qt;
        prev_turn = turn;
        uint32_t ok = 1;
        if (lane == 0) ok = turn_wait(turn, 4 * kv_tile, abort_flag, args.status) ? 1u : 0u;
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) {
          if (lane == 0) {
            atomicExch(args.status, FSB_ERR_WAIT_TIMEOUT_PEER);
            *abort_flag = 1;
          }
          prev_turn = nullptr;
          break;
        }
      }
      float* base = args.dq_acc + static_cast<long long>(row_base + walk.qt * BQ) * ldq + (hk * G + walk.g) * HD + d;
#pragma unroll
      for (int c = 0; c < 32; ++c) red_add_f32(base + c * ldq, __uint_as_float(v0[c]) * sc);
#pragma unroll
      for (int c = 0; c < 32; ++c) red_add_f32(base + (32 + c) * ldq, __uint_as_float(v1[c]) * sc);
      walk.next(qt_first, n_qt, G, args.heads_inner);
    }
    if (prev_turn != nullptr) {   // the last tile's turn
      __syncwarp();
      if (lane == 0) {
        __threadfence();
        atomicAdd(prev_turn, 1);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    if (*abort_flag) {
      const unsigned long long t0 = clock64();
      while (clock64() - t0 < 2000000ull) {
      }
    }
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// delta[b, h, s] = sum_d O * dO   (one warp per (row, head))
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o,
                                  float* __restrict__ delta, int B, int S, int H, long long ldo,
                                  long long lddo) {
  const long long w = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long long total = static_cast<long long>(B) * S * H;
  if (w >= total) return;
  const int h = w % H;
  const long long row = w / H;  // b*S + s
  const __nv_bfloat162* po = reinterpret_cast<const __nv_bfloat162*>(o + row * ldo + h * HD) + lane * 2;
  const __nv_bfloat162* pd = reinterpret_cast<const __nv_bfloat162*>(d_o + row * lddo + h * HD) + lane * 2;
  float acc = 0.f;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const float2 a = __bfloat1622float2(po[i]), c = __bfloat1622float2(pd[i]);
    acc += a.x * c.x + a.y * c.y;
  }
  acc = warp_sum(acc);
  if (lane == 0) {
    const long long bb = row / S, ss = row % S;
    delta[(bb * H + h) * S + ss] = acc;
  }
}

}  // namespace

// dq_acc: fp32 [B*S, Hq*128], must be zero on entry. dk/dv: bf16 [B*S, Hkv*128] slices with row
// strides lddk/lddv. delta: fp32 scratch [B, Hq, S] (written here). turns: null, or B*Hq*(S/64) + 1 zeroed
// ints, which selects the ordered (bitwise reproducible) accumulation of dQ. heads_inner: the walk order
// (see TileWalk); the ordered mode wants 1.
FSB_API int fsb_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o,
                         const float* lse, float* delta, float* dq_acc, int* turns, int heads_inner, void* dk, void* dv, int B, int S,
                         int Hq, int Hkv, long long ldq, long long ldk, long long ldv, long long ldo,
                         long long lddo, long long lddk, long long lddv, float softmax_scale,
                         int* status, cudaStream_t stream) {
  if (S % BKV != 0 || Hq % Hkv != 0 || B <= 0 || (lddk % 8) || (lddv % 8)) return FSB_ERR_BAD_ARG;
  if (static_cast<long long>(B) * Hq * S >= (1ll << 31)) return FSB_ERR_TOO_LARGE;
  CUtensorMap mq, mk, mv, mdo;
  const uint64_t rows = static_cast<uint64_t>(B) * S;
  int rc = fsb_make_tmap_2d(&mq, q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, rows, static_cast<uint64_t>(Hq) * HD, ldq, BQ, 64);
  if (rc != FSB_OK) return rc;
  rc = fsb_make_tmap_2d(&mdo, d_o, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, rows, static_cast<uint64_t>(Hq) * HD, lddo, BQ, 64);
  if (rc != FSB_OK) return rc;
  rc = fsb_make_tmap_2d(&mk, k, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, rows, static_cast<uint64_t>(Hkv) * HD, ldk, BKV, 64);
  if (rc != FSB_OK) return rc;
  rc = fsb_make_tmap_2d(&mv, v, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, rows, static_cast<uint64_t>(Hkv) * HD, ldv, BKV, 64);
  if (rc != FSB_OK) return rc;
  {
    const long long warps = static_cast<long long>(B) * S * Hq;
    const int threads = 256;
    const long long blocks = (warps * 32 + threads - 1) / threads;
    attn_delta_kernel<<<static_cast<unsigned>(blocks), threads, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(o), static_cast<const __nv_bfloat16*>(d_o), delta, B, S, Hq, ldo, lddo);
  }
  if (cudaFuncSetAttribute(attn_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BWD) != cudaSuccess)
    return FSB_ERR_LAUNCH;
  BwdArgs a;
  a.S = S; a.Hq = Hq; a.Hkv = Hkv;
  a.scale = softmax_scale;
  a.scale_log2 = softmax_scale * 1.4426950408889634f;
  a.lse = lse; a.delta = delta; a.dq_acc = dq_acc; a.turns = turns; a.heads_inner = heads_inner ? 1 : 0;
  a.dk = static_cast<__nv_bfloat16*>(dk); a.lddk = lddk;
  a.dv = static_cast<__nv_bfloat16*>(dv); a.lddv = lddv;
  a.status = status;
  dim3 grid(Hkv * B, S / BKV, 1);
  attn_bwd_kernel<<<grid, THREADS, SMEM_BWD, stream>>>(mq, mk, mv, mdo, a);
  return cudaGetLastError() == cudaSuccess ? FSB_OK : FSB_ERR_LAUNCH;
}
