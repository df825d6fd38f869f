// Tensor-core GEMM on CTA pairs with wide tiles: 256 columns j x W rows i per pair, W up to 512.
//
// What wider tiles buy: a 256 x W tile moves (128 + W / 2) * 128 operand bytes per CTA and k-block for 2 W clocks
// of MMA work -- at W = 512 that is 25 % fewer bytes per FLOP than the 256 x 256 tiles of gemm_tc2.cuh (measured:
// L2 throughput 30 % instead of 43 %, DRAM 13 % instead of 16 %) -- and half as many tiles.  What they do not buy on
// B200 is a faster mainloop: the FP8 mainloop is power-bound there (under ncu this kernel runs at a higher SM clock
// with a proportionally less busy tensor pipe; clock x pipe-active is the same for both kernels), so the gain is
// the 2 to 7 % that fewer bytes and fewer tile transitions are worth on long-K problems.
//
// Price: the two W / 2-column accumulators (one N = W / 2 MMA each per 32 bytes of K) fill the 512 columns
// of tensor memory, so there is no second buffer and the epilogue of a tile is not hidden behind the next
// tile's mainloop (the TMA ring keeps filling meanwhile).  That pays when K is long next to the epilogue;
// the launcher chooses between this kernel, its width, and the double-buffered 256 x 256 kernel from a
// tuned table and a small cost model.
//
// Roles, barriers, bounded waits, pairing and the common exit are those of gemm_tc2.cuh.  No load is
// multicast: each CTA fetches its own 128 rows of op(B)^T and its own two boxes of W / 4 rows of op(A).
#pragma once
#include "gemm_tc2.cuh"

namespace e5b {
namespace tc {

constexpr int W_MAX = 512;
constexpr int W_SMEM_LIMIT = 232448 - 2048;   // dynamic shared memory the kernel may use (ring + barriers + alignment)

// Instruction descriptors for items of width W, W / 2 and W / 4 (N = half of that each).
struct WideDescs { uint32_t idesc[3]; };

// map_i[0..2]: op(A) with boxes of W / 4, W / 8, W / 16 rows (whole tiles, half and quarter slices of the last round).
template <int KIND, int DT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
gemm_tc_pairw_kernel(const __grid_constant__ CUtensorMap map_i0, const __grid_constant__ CUtensorMap map_j,
                     const __grid_constant__ CUtensorMap map_i1, const __grid_constant__ CUtensorMap map_i2, int m, int n,
                     int k_bytes, int W, int stages, int slices, WideDescs wd, OutDesc o, EpiMode md) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t ring = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t stage_bytes = (uint32_t)P_HALF_BYTES + (uint32_t)(W / 2) * STAGE_K_BYTES;
  uint8_t *after_ring = smem_raw + (ring - smem_u32(smem_raw)) + stages * stage_bytes;
  uint64_t *bars = reinterpret_cast<uint64_t *>(after_ring);   // full[8], empty[8], acc_full, acc_empty
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 18);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
  const uint32_t bar0 = smem_u32(bars);
  const auto full_bar = [&](int s) { return bar0 + 8u * s; };
  const auto empty_bar = [&](int s) { return bar0 + 8u * (8 + s); };
  const uint32_t acc_full = bar0 + 8u * 16, acc_empty = bar0 + 8u * 17;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();
  const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
  const int tiles_i = (m + W - 1) / W, tiles_j = (n + P_TILE - 1) / P_TILE, tiles = tiles_i * tiles_j;
  const int kblocks = (k_bytes + STAGE_K_BYTES - 1) / STAGE_K_BYTES;

  // Work items as in the 256 x 256 kernel: whole tiles dealt round-robin; the tiles of a sparsely filled last
  // round are cut into f = slices (1, 2 or 4) pieces of W / f rows.  level = log2(f) of an item selects its
  // tensor map and instruction descriptor.
  const int full_items = (tiles / pairs) * pairs, rest = tiles - full_items;
  const int f = rest > 0 ? slices : 1;
  const int items = full_items + f * rest;
  const auto item_at = [&](int item, int &i0, int &j0, int &w, int &level) {
    int tile = item, sub = 0;
    w = W;
    level = 0;
    if (item >= full_items) { const int h = item - full_items; tile = full_items + h / f; sub = h % f; w = W / f; level = f >> 1; }
    int ti, tj;
    tile_coords(tile, tiles_i, tiles_j, ti, tj);
    i0 = ti * W + sub * w;
    j0 = tj * P_TILE;
  };

  if (threadIdx.x == 32) { prefetch_map(&map_i0); prefetch_map(&map_j); prefetch_map(&map_i1); prefetch_map(&map_i2); }
  if (threadIdx.x == 0) {
    for (int s = 0; s < 8; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    mbar_init(acc_full, 1);
    mbar_init(acc_empty, 2 * EPI_WARPS);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(tmem_slot), 512);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t peer_abort = map_to_rank(smem_u32(const_cast<int *>(abort_flag)), rank ^ 1u);   // the other CTA's abort flag

  if (warp == 0) {
    // ---------------- TMA producer (both CTAs) ----------------
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int t = pair; t < items && ok; t += pairs) {
        int i0, j0, w, level;
        item_at(t, i0, j0, w, level);
        const int h = w / 4;                       // rows per box of op(A)
        const CUtensorMap *mi = level == 0 ? &map_i0 : (level == 1 ? &map_i1 : &map_i2);
        const uint32_t pair_bytes = 2u * (P_HALF_BYTES + (uint32_t)(w / 2) * STAGE_K_BYTES);
        const int jr = j0 + (int)rank * 128;
        const int ia = i0 + (int)rank * h, ib = i0 + w / 2 + (int)rank * h;   // this CTA's rows of the two MMAs' N sides
        const bool backwards = ((t / pairs) & 1) != 0;
        for (int kq = 0; kq < kblocks; ++kq) {
          const int kb = backwards ? kblocks - 1 - kq : kq;
          if (!mbar_wait(empty_bar(s), ph ^ 1u, abort_flag, (1u << 24) | (uint32_t)kb, peer_abort)) { ok = false; break; }
          const uint32_t lead_full = map_to_rank(full_bar(s), 0);
          if (rank == 0) mbar_expect_tx(full_bar(s), pair_bytes);
          const uint32_t sj = ring + s * stage_bytes, si = sj + P_HALF_BYTES;
          const int kc = kb * (KIND == 0 ? STAGE_K_BYTES : STAGE_K_BYTES / 2);
          tma_load_2d_pair(sj, &map_j, kc, jr, lead_full);
          tma_load_2d_pair(si, mi, kc, ia, lead_full);
          tma_load_2d_pair(si + (uint32_t)h * STAGE_K_BYTES, mi, kc, ib, lead_full);
          if (++s == stages) { s = 0; ph ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (leader CTA only) ----------------
    if (lane == 0 && rank == 0) {
      int s = 0;
      uint32_t ph = 0, lt = 0;
      bool ok = true;
      for (int t = pair; t < items && ok; t += pairs, ++lt) {
        int i0, j0, w, level;
        item_at(t, i0, j0, w, level);
        const uint32_t idesc_t = level == 0 ? wd.idesc[0] : (level == 1 ? wd.idesc[1] : wd.idesc[2]);
        const uint32_t box_step = ((uint32_t)(w / 4) * STAGE_K_BYTES) >> 4;   // second box, in descriptor address units
        if (!mbar_wait(acc_empty, (lt & 1u) ^ 1u, abort_flag, (2u << 24) | 0xFFFFu, peer_abort)) { ok = false; break; }
        tc_fence_after();
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(full_bar(s), ph, abort_flag, (2u << 24) | (uint32_t)kb, peer_abort)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sj = ring + s * stage_bytes, si = sj + P_HALF_BYTES;
          const uint64_t dj = kmajor_sw128_desc(sj), di = kmajor_sw128_desc(si);
#pragma unroll
          for (int ks = 0; ks < STAGE_K_BYTES / MMA_K_BYTES; ++ks) {
            mma_ss_pair<KIND>(tmem_base, dj + 2u * ks, di + 2u * ks, idesc_t, (kb | ks) != 0);
            mma_ss_pair<KIND>(tmem_base + 256u, dj + 2u * ks, di + box_step + 2u * ks, idesc_t, (kb | ks) != 0);
          }
          mma_commit_pair(empty_bar(s));
          mma_commit_pair(map_to_rank(empty_bar(s), 1));
          if (++s == stages) { s = 0; ph ^= 1u; }
        }
        if (ok) {
          mma_commit_pair(acc_full);
          mma_commit_pair(map_to_rank(acc_full, 1));
        }
      }
    }
  } else {
    // ---------------- epilogue (both CTAs): own 128 TMEM lanes; warps 2-5 drain the first accumulator, 6-9 the second ----------------
    const int quad = warp & 3, q = (warp - 2) >> 2;
    const OutScalars r = out_begin(o);
    const float as_const = __fmul_rn(o.alpha, o.sa_vec ? 1.f : ld_or_one(o.sa));
    const float sb_const = o.sb_vec ? 1.f : ld_or_one(o.sb);
    float mx = 0.f;
    uint32_t lt = 0;
    bool ok = true;
    for (int t = pair; t < items && ok; t += pairs, ++lt) {
      int i0, j0, w, level;
      item_at(t, i0, j0, w, level);
      ok = mbar_wait(acc_full, lt & 1u, abort_flag, (3u << 24) | (uint32_t)warp, peer_abort);
      ok = __all_sync(0xFFFFFFFFu, ok);
      if (!ok) break;
      tc_fence_after();
      const int j = j0 + (int)rank * 128 + quad * 32 + lane;
      const bool col_ok = j < n;
      const float sbj = col_ok && o.sb_vec ? o.sb[j] : sb_const;
      const uint32_t t_lane = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)q * 256u;
      const int ibase = i0 + q * (w / 2);
      const int lim = m < ibase + w / 2 ? m : ibase + w / 2;     // rows of this accumulator that exist
      for (int c0 = 0; c0 < w / 2; c0 += 32) {
        if (ibase + c0 >= lim) break;   // warp-uniform
        float acc[32];
        tmem_ld32(t_lane + c0, acc);
        if (col_ok) mx = fmaxf(mx, drain32<DT>(o, r, md, acc, ibase + c0, j, lim, as_const, sbj));
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_rank(acc_empty, 0));
      bcast_block<DT>(o, j0 + (int)rank * 128 + quad * 32, n, ibase, lim);   // e5b_gemm_bcast: this warp's block goes to the peers
    }
    if (o.amax) {
      mx = warp_max(mx);
      if (lane == 0) amax_publish(o.amax, mx);
    }
  }

  // common exit: the CTA meets, then the pair meets, then tensor memory is released by both
  tc_fence_before();
  __syncthreads();
  if (*abort_flag && threadIdx.x == 0) {
    const unsigned long long t0 = clock64();
    while ((unsigned long long)(clock64() - t0) < 2000000ull) { }
  }
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, 512);
  }
}

struct WidePlan { int W, stages, slices, smem; };

// Stages that fit, slices the width allows for `rest` tiles left over after the full rounds.
inline WidePlan wide_plan(int W, int tiles, int pairs) {
  WidePlan p;
  p.W = W;
  const int stage_bytes = P_HALF_BYTES + (W / 2) * STAGE_K_BYTES;
  p.stages = (W_SMEM_LIMIT - 1024 - 256) / stage_bytes;
  if (p.stages > 8) p.stages = 8;
  p.smem = p.stages * stage_bytes + 1024 + 256;
  const int rest = tiles % pairs;
  p.slices = 1;
  // Halves only: a quarter slice would run two MMAs of N = W / 8 per 32 bytes of K, and MMAs that narrow cost about
  // as much as N = 128 ones (measured: 96-wide slices of W = 384 took 1170 clocks per k-block instead of 270).
  if (rest > 0 && opt(OPT_TC_SPLIT) != 0 && W % 64 == 0 && 2 * rest <= pairs) p.slices = 2;
  return p;
}

template <int KIND, int DT>
static cudaError_t launch_pairw_cfg(const CUtensorMap *mi, const CUtensorMap &mj, int m, int n, int k_bytes, const WidePlan &p,
                                    const WideDescs &wd, const OutDesc &o, const EpiMode &md, int pairs, cudaStream_t s) {
  static SmemOptIn optin;
  if (const cudaError_t e = optin.ensure(gemm_tc_pairw_kernel<KIND, DT>, W_SMEM_LIMIT)) return e;
  note_route(ROUTE_TC_PAIR_WIDE);
  gemm_tc_pairw_kernel<KIND, DT><<<2 * pairs, THREADS, p.smem, s>>>(mi[0], mj, mi[1], mi[2], m, n, k_bytes, p.W, p.stages,
                                                                     p.slices, wd, o, md);
  return cudaGetLastError();
}

template <int KIND>
static cudaError_t launch_pairw(const CUtensorMap *mi, const CUtensorMap &mj, int m, int n, int k_bytes, const WidePlan &p,
                                const WideDescs &wd, const OutDesc &o, const EpiMode &md, int pairs, cudaStream_t s) {
  switch (o.d_dtype) {
    case E5MA_BF16: return launch_pairw_cfg<KIND, E5MA_BF16>(mi, mj, m, n, k_bytes, p, wd, o, md, pairs, s);
    case E5MA_FP32: return launch_pairw_cfg<KIND, E5MA_FP32>(mi, mj, m, n, k_bytes, p, wd, o, md, pairs, s);
    case E5MA_FP16: return launch_pairw_cfg<KIND, E5MA_FP16>(mi, mj, m, n, k_bytes, p, wd, o, md, pairs, s);
    case E5MA_E5M2: return launch_pairw_cfg<KIND, E5MA_E5M2>(mi, mj, m, n, k_bytes, p, wd, o, md, pairs, s);
    default: return launch_pairw_cfg<KIND, E5MA_E4M3>(mi, mj, m, n, k_bytes, p, wd, o, md, pairs, s);
  }
}

}  // namespace tc
}  // namespace e5b
