// Causal flash-attention backward for sm_100a (head_dim 128, GQA), bf16.
//
// One CTA owns a 128-row key/value tile of one KV head and walks every query
// tile (64 rows) at or below the diagonal, for each query head of the group.
// Everything is computed transposed so that the kv index is the MMA M dimension
// (= TMEM lane = softmax thread) and no operand needs a transpose copy:
//   S^T  = K Q^T          A = K  (K-major)      B = Q  (K-major)        -> TMEM buf[b][ 0: 64)
//   dP^T = V dO^T         A = V  (K-major)      B = dO (K-major)        -> TMEM buf[b][64:128)
//   P^T  = exp2(S^T*c - lse), dS^T = P^T (dP^T - delta) * scale         threads -> bf16 smem
//   dV  += P^T  dO        A = P^T  (K-major)    B = dO (same tile, MN-major)
//   dK  += dS^T Q         A = dS^T (K-major)    B = Q  (same tile, MN-major)
//   dQ^T = K^T dS         A = K (MN-major)      B = dS^T (same tile, MN-major) -> TMEM buf[b][0:64)
// dQ^T is transposed through shared memory and added into a fp32 [B*S, Hq*128] accumulator
// by one bulk tensor reduce-add per query tile (the copy engine does the read-modify-write at L2).
// TMEM: two (S^T|dP^T) buffers (256 columns) + dV (128) + dK (128) = 512 columns.
#include "common.cuh"

namespace {
using namespace fsb;

constexpr int HD = 128;
constexpr int BKV = 128;
constexpr int BQ = 64;
constexpr int KV_TILE_BYTES = BKV * HD * 2;  // 32 KB, two chunks of 16 KB
constexpr int Q_TILE_BYTES = BQ * HD * 2;    // 16 KB, two chunks of 8 KB
constexpr int PT_BYTES = BKV * BQ * 2;       // 16 KB
constexpr int DQ_BYTES = BQ * HD * 4;           // 32 KB fp32 staging tile [64 q][128 d]
constexpr int SMEM_BWD = 2 * KV_TILE_BYTES + 2 * 2 * Q_TILE_BYTES + 2 * PT_BYTES + DQ_BYTES + 1024 + 4096 + 256;
constexpr int THREADS = 320;  // warp 0 TMA, warp 1 MMA, warps 2..9 compute (two per TMEM lane quarter)

struct BwdArgs {
  int S, Hq, Hkv;
  float scale_log2, scale;
  const float* lse;    // [B, Hq, S]
  const float* delta;  // [B, Hq, S]
  float* dq_acc;       // [B*S, Hq*128] fp32, zero-initialised
  __nv_bfloat16* dk;
  long long lddk;
  __nv_bfloat16* dv;
  long long lddv;
  int* status;
};

__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&o)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr),
      "r"(o[0]), "r"(o[1]), "r"(o[2]), "r"(o[3]), "r"(o[4]), "r"(o[5]), "r"(o[6]), "r"(o[7]), "r"(o[8]),
      "r"(o[9]), "r"(o[10]), "r"(o[11]), "r"(o[12]), "r"(o[13]), "r"(o[14]), "r"(o[15]), "r"(o[16]),
      "r"(o[17]), "r"(o[18]), "r"(o[19]), "r"(o[20]), "r"(o[21]), "r"(o[22]), "r"(o[23]), "r"(o[24]),
      "r"(o[25]), "r"(o[26]), "r"(o[27]), "r"(o[28]), "r"(o[29]), "r"(o[30]), "r"(o[31])
      : "memory");
}

__global__ void __launch_bounds__(THREADS, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do,
                const __grid_constant__ CUtensorMap map_dq, const BwdArgs args) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sK = smem;
  uint8_t* sV = sK + KV_TILE_BYTES;
  uint8_t* sQ = sV + KV_TILE_BYTES;          // [2][Q_TILE_BYTES]
  uint8_t* sDO = sQ + 2 * Q_TILE_BYTES;      // [2][Q_TILE_BYTES]
  uint8_t* sPT = sDO + 2 * Q_TILE_BYTES;     // P^T
  uint8_t* sDST = sPT + PT_BYTES;            // dS^T
  // per softmax warp: [2 stages][64 lse | 64 delta] (each warp stages its own copy, so the
  // warps never have to meet at a CTA-wide barrier inside the loop)
  float* sDQ = reinterpret_cast<float*>(sDST + PT_BYTES);   // [64 q][128 d] fp32
  float* s_stats = reinterpret_cast<float*>(sDST + PT_BYTES + DQ_BYTES);
  uint64_t* bars = reinterpret_cast<uint64_t*>(sDST + PT_BYTES + DQ_BYTES + 4096);
  uint64_t* kv_full = bars;          // 1
  uint64_t* qdo_full = bars + 1;     // [2]
  uint64_t* qdo_empty = bars + 3;    // [2]
  uint64_t* sdp_full = bars + 5;     // [2]
  uint64_t* buf_empty = bars + 7;    // [2]  threads drained dQ^T from TMEM buffer b
  uint64_t* pds_full = bars + 9;     // threads wrote P^T / dS^T
  uint64_t* pds_empty = bars + 10;   // MMAs finished reading P^T / dS^T
  uint64_t* dq_full = bars + 11;     // [2]
  uint64_t* all_done = bars + 13;
  uint64_t* sdq_free = bars + 14;     // the previous reduce-add has finished reading sDQ
  uint64_t* sdq_written = bars + 15;  // all four warps have written their part of sDQ
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // x = (kv head, batch) so that CTAs are handed out tile by tile: kv tile 0 has the most
  // query tiles below the diagonal, so ascending y is longest-job-first.
  const int kv_tile = blockIdx.y;
  const int hk = blockIdx.x % args.Hkv, b = blockIdx.x / args.Hkv;
  const int G = args.Hq / args.Hkv;
  const int kv0 = kv_tile * BKV;
  const int row_base = b * args.S;
  const int qt_first = kv0 / BQ;
  const int n_qt = args.S / BQ - qt_first;   // query tiles per head
  const int n_it = n_qt * G;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&qdo_full[i], 1);
      mbar_init(&qdo_empty[i], 1);
      mbar_init(&sdp_full[i], 1);
      mbar_init(&buf_empty[i], 8);
      mbar_init(&dq_full[i], 1);
    }
    mbar_init(pds_full, 8);
    mbar_init(pds_empty, 1);
    mbar_init(all_done, 1);
    mbar_init(sdq_free, 1);
    mbar_init(sdq_written, 8);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
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
      for (int it = 0; it < n_it; ++it) {
        const int s = it & 1;
        const uint32_t ph = (it >> 1) & 1;
        const int g = it / n_qt, qt = qt_first + it % n_qt;
        const int h = hk * G + g;
        if (!mbar_wait(&qdo_empty[s], ph ^ 1, abort_flag)) {
          atomicExch(args.status, FSB_ERR_WAIT_TIMEOUT_EMPTY);
          *abort_flag = 1;
          break;
        }
        mbar_expect_tx(&qdo_full[s], 2 * Q_TILE_BYTES);
        uint8_t* q = sQ + s * Q_TILE_BYTES;
        uint8_t* d = sDO + s * Q_TILE_BYTES;
        const int row = row_base + qt * BQ;
        tma_load_2d(q, &map_q, &qdo_full[s], h * HD, row);
        tma_load_2d(q + Q_TILE_BYTES / 2, &map_q, &qdo_full[s], h * HD + 64, row);
        tma_load_2d(d, &map_do, &qdo_full[s], h * HD, row);
        tma_load_2d(d + Q_TILE_BYTES / 2, &map_do, &qdo_full[s], h * HD + 64, row);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc_sdp = make_idesc(BKV, BQ, 1, 1, 0, 0);   // M=128 kv, N=64 q
      const uint32_t idesc_dkv = make_idesc(BKV, HD, 1, 1, 0, 1);   // M=128 kv, N=128 d, B MN-major
      const uint32_t idesc_dq = make_idesc(HD, BQ, 1, 1, 1, 1);     // M=128 d,  N=64 q, both MN-major
      const uint32_t k_addr = smem_u32(sK), v_addr = smem_u32(sV);
      const uint32_t pt_addr = smem_u32(sPT), dst_addr = smem_u32(sDST);
      bool ok = mbar_wait(kv_full, 0, abort_flag);

      auto issue_sdp = [&](int it) -> bool {
        const int s = it & 1;
        const uint32_t ph = (it >> 1) & 1;
        if (!mbar_wait(&qdo_full[s], ph, abort_flag) || !mbar_wait(&buf_empty[s], ph ^ 1, abort_flag))
          return false;
        tc_fence_after();
        const uint32_t q_addr = smem_u32(sQ + s * Q_TILE_BYTES);
        const uint32_t do_addr = smem_u32(sDO + s * Q_TILE_BYTES);
        const uint32_t t_s = tmem_base + s * 128;
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint32_t ka = k_addr + (k >> 2) * (KV_TILE_BYTES / 2) + (k & 3) * 32;
          const uint32_t qa = q_addr + (k >> 2) * (Q_TILE_BYTES / 2) + (k & 3) * 32;
          umma_f16(t_s, make_smem_desc_sw128(ka, 16, 1024), make_smem_desc_sw128(qa, 16, 1024),
                   idesc_sdp, k != 0);
        }
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint32_t va = v_addr + (k >> 2) * (KV_TILE_BYTES / 2) + (k & 3) * 32;
          const uint32_t da = do_addr + (k >> 2) * (Q_TILE_BYTES / 2) + (k & 3) * 32;
          umma_f16(t_s + 64, make_smem_desc_sw128(va, 16, 1024), make_smem_desc_sw128(da, 16, 1024),
                   idesc_sdp, k != 0);
        }
        umma_commit(&sdp_full[s]);
        return true;
      };

      if (ok && n_it > 0) ok = issue_sdp(0);
      for (int it = 0; it < n_it && ok; ++it) {
        const int s = it & 1;
        if (it + 1 < n_it) {
          ok = issue_sdp(it + 1);
          if (!ok) break;
        }
        if (!mbar_wait(pds_full, it & 1, abort_flag)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t q_addr = smem_u32(sQ + s * Q_TILE_BYTES);
        const uint32_t do_addr = smem_u32(sDO + s * Q_TILE_BYTES);
        // dV += P^T dO ; dK += dS^T Q   (K = 64 queries, 4 steps; B tiles read MN-major:
        // d chunks 8 KB apart (LBO), 8-query groups 1 KB apart (SBO), 16 queries = 2 KB)
#pragma unroll
        for (int k = 0; k < BQ / 16; ++k) {
          umma_f16(tmem_dv, make_smem_desc_sw128(pt_addr + k * 32, 16, 1024),
                   make_smem_desc_sw128(do_addr + k * 2048, Q_TILE_BYTES / 2, 1024), idesc_dkv,
                   (it | k) != 0);
        }
#pragma unroll
        for (int k = 0; k < BQ / 16; ++k) {
          umma_f16(tmem_dk, make_smem_desc_sw128(dst_addr + k * 32, 16, 1024),
                   make_smem_desc_sw128(q_addr + k * 2048, Q_TILE_BYTES / 2, 1024), idesc_dkv,
                   (it | k) != 0);
        }
        // dQ^T = K^T dS: A = K read MN-major (d chunks 16 KB apart, 8-kv groups 1 KB apart),
        // B = dS^T read MN-major (a single 64-query group), K = 128 kv in 8 steps of 2 KB.
#pragma unroll
        for (int k = 0; k < BKV / 16; ++k) {
          umma_f16(tmem_base + s * 128, make_smem_desc_sw128(k_addr + k * 2048, KV_TILE_BYTES / 2, 1024),
                   make_smem_desc_sw128(dst_addr + k * 2048, PT_BYTES, 1024), idesc_dq, k != 0);
        }
        umma_commit(&qdo_empty[s]);
        umma_commit(pds_empty);
        umma_commit(&dq_full[s]);
      }
      if (ok) {
        umma_commit(all_done);
      } else {
        atomicExch(args.status, FSB_ERR_WAIT_TIMEOUT_FULL);
        *abort_flag = 1;
      }
    }
  } else {
    // ------------------------------------------------------------ softmax / drain warps
    // Two warps share each TMEM lane quarter and split the columns between them: every element of
    // the backward pass is independent (no row reductions), so the split needs no exchange.
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;    // 0: columns [0,32) of a 64-wide tile, 1: columns [32,64)
    const int r = quarter * 32 + lane;   // kv row inside the tile (S^T, dP^T, dK, dV) or d (dQ^T)
    const int kv_row = kv0 + r;
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    const float LOG2E = 1.4426950408889634f;
    bool ok = true;

    // dQ^T (lane = d, column = q) -> sDQ[q][d] -> one bulk reduce-add into dq_acc.
    auto drain_dq = [&](int it) -> bool {
      const int s = it & 1;
      const uint32_t ph = (it >> 1) & 1;
      if (!mbar_wait(&dq_full[s], ph, abort_flag)) return false;
      tc_fence_after();
      const int g = it / n_qt, qt = qt_first + it % n_qt;
      const int h = hk * G + g;
      // the previous tile's reduce must have finished reading sDQ before it is overwritten
      // (mbarriers with bounded waits rather than a CTA barrier: a warp that gave up must not
      // leave the others waiting for it)
      const uint32_t dph = static_cast<uint32_t>(it) & 1;
      if (threadIdx.x == 64) {
        tma_store_wait_read0();
        mbar_arrive(sdq_free);
      }
      if (!mbar_wait(sdq_free, dph, abort_flag)) return false;
      {
        const int c0 = half * 32;
        uint32_t v[32];
        tmem_ld_32x32(tmem_base + lane_off + s * 128 + c0, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) sDQ[(c0 + i) * HD + r] = __uint_as_float(v[i]);
      }
      tc_fence_before();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&buf_empty[s]);
        mbar_arrive(sdq_written);
      }
      if (threadIdx.x == 64) {
        if (!mbar_wait(sdq_written, dph, abort_flag)) return false;
        tma_reduce_add_2d(&map_dq, sDQ, h * HD, row_base + qt * BQ);
        tma_store_commit();
      }
      return true;
    };

    for (int it = 0; it < n_it; ++it) {
      const int s = it & 1;
      const uint32_t ph = (it >> 1) & 1;
      const int g = it / n_qt, qt = qt_first + it % n_qt;
      const int h = hk * G + g;
      const int q0 = qt * BQ;
      // stage this tile's lse / delta rows (64 each) in this warp's private slot
      float* s_lse = s_stats + ((warp - 2) * 2 + s) * 64;   // this warp's 32 queries: lse | delta
      float* s_delta = s_lse + 32;
      {
        const long long off = (static_cast<long long>(b) * args.Hq + h) * args.S + q0 + half * 32;
        s_lse[lane] = args.lse[off + lane] * LOG2E;
        s_delta[lane] = args.delta[off + lane];
        __syncwarp();
      }
      if (!mbar_wait(&sdp_full[s], ph, abort_flag)) {
        ok = false;
        break;
      }
      tc_fence_after();
      if (it > 0 && !mbar_wait(pds_empty, (it - 1) & 1, abort_flag)) {
        ok = false;
        break;
      }
      const bool diag = q0 < kv0 + BKV;  // some (kv, q) pairs of this tile are above the diagonal
      uint8_t* prow = sPT + r * 128;
      uint8_t* drow = sDST + r * 128;
      {
        const int c0 = half * 32;
        uint32_t sv[32], dp[32];
        tmem_ld_32x32(tmem_base + lane_off + s * 128 + c0, sv);
        tmem_ld_32x32(tmem_base + lane_off + s * 128 + 64 + c0, dp);
        tmem_ld_wait();
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          float p[8], d[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int c = u * 8 + i;
            const int qi = c0 + c;
            float pv = exp2f(__uint_as_float(sv[c]) * args.scale_log2 - s_lse[c]);
            if (diag && kv_row > q0 + qi) pv = 0.f;
            p[i] = pv;
            d[i] = pv * (__uint_as_float(dp[c]) - s_delta[c]) * args.scale;
          }
          uint4 pk, dk;
          pk.x = pack_bf16x2(p[0], p[1]); pk.y = pack_bf16x2(p[2], p[3]);
          pk.z = pack_bf16x2(p[4], p[5]); pk.w = pack_bf16x2(p[6], p[7]);
          dk.x = pack_bf16x2(d[0], d[1]); dk.y = pack_bf16x2(d[2], d[3]);
          dk.z = pack_bf16x2(d[4], d[5]); dk.w = pack_bf16x2(d[6], d[7]);
          const int unit = ((c0 >> 3) + u) ^ (r & 7);
          *reinterpret_cast<uint4*>(prow + (unit << 4)) = pk;
          *reinterpret_cast<uint4*>(drow + (unit << 4)) = dk;
        }
      }
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(pds_full);
      if (it > 0 && !drain_dq(it - 1)) {
        ok = false;
        break;
      }
    }
    if (ok && n_it > 0) ok = drain_dq(n_it - 1);
    if (threadIdx.x == 64) tma_store_wait_all();
    if (ok && mbar_wait(all_done, 0, abort_flag)) {
      tc_fence_after();
      __nv_bfloat16* dkrow = args.dk + static_cast<long long>(row_base + kv_row) * args.lddk + hk * HD;
      __nv_bfloat16* dvrow = args.dv + static_cast<long long>(row_base + kv_row) * args.lddv + hk * HD;
#pragma unroll 1
      for (int c0 = half * 64; c0 < half * 64 + 64; c0 += 32) {
        uint32_t a[32], c[32];
        tmem_ld_32x32(tmem_dk + lane_off + c0, a);
        tmem_ld_32x32(tmem_dv + lane_off + c0, c);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; i += 8) {
          uint4 x, y;
          x.x = pack_bf16x2(__uint_as_float(a[i]), __uint_as_float(a[i + 1]));
          x.y = pack_bf16x2(__uint_as_float(a[i + 2]), __uint_as_float(a[i + 3]));
          x.z = pack_bf16x2(__uint_as_float(a[i + 4]), __uint_as_float(a[i + 5]));
          x.w = pack_bf16x2(__uint_as_float(a[i + 6]), __uint_as_float(a[i + 7]));
          y.x = pack_bf16x2(__uint_as_float(c[i]), __uint_as_float(c[i + 1]));
          y.y = pack_bf16x2(__uint_as_float(c[i + 2]), __uint_as_float(c[i + 3]));
          y.z = pack_bf16x2(__uint_as_float(c[i + 4]), __uint_as_float(c[i + 5]));
          y.w = pack_bf16x2(__uint_as_float(c[i + 6]), __uint_as_float(c[i + 7]));
          *reinterpret_cast<uint4*>(dkrow + c0 + i) = x;
          *reinterpret_cast<uint4*>(dvrow + c0 + i) = y;
        }
      }
    } else if (lane == 0) {
      atomicExch(args.status, FSB_ERR_WAIT_TIMEOUT_TMEM_FULL);
      *abort_flag = 1;
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
// strides lddk/lddv. delta: fp32 scratch [B, Hq, S] (written here).
FSB_API int fsb_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o,
                         const float* lse, float* delta, float* dq_acc, void* dk, void* dv, int B, int S,
                         int Hq, int Hkv, long long ldq, long long ldk, long long ldv, long long ldo,
                         long long lddo, long long lddk, long long lddv, float softmax_scale,
                         int* status, cudaStream_t stream) {
  if (S % BKV != 0 || Hq % Hkv != 0 || B <= 0 || (lddk % 8) || (lddv % 8)) return FSB_ERR_BAD_ARG;
  CUtensorMap mq, mk, mv, mdo, mdq;
  const uint64_t rows = static_cast<uint64_t>(B) * S;
  int rc0 = fsb_make_tmap_2d_plain(&mdq, dq_acc, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, rows,
                                   static_cast<uint64_t>(Hq) * HD, static_cast<uint64_t>(Hq) * HD, BQ, HD);
  if (rc0 != FSB_OK) return rc0;
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
  a.lse = lse; a.delta = delta; a.dq_acc = dq_acc;
  a.dk = static_cast<__nv_bfloat16*>(dk); a.lddk = lddk;
  a.dv = static_cast<__nv_bfloat16*>(dv); a.lddv = lddv;
  a.status = status;
  dim3 grid(Hkv * B, S / BKV, 1);
  attn_bwd_kernel<<<grid, THREADS, SMEM_BWD, stream>>>(mq, mk, mv, mdo, mdq, a);
  return cudaGetLastError() == cudaSuccess ? FSB_OK : FSB_ERR_LAUNCH;
}
