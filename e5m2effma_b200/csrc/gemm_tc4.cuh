// Tensor-core GEMM on CTA pairs for mixed FP8 x BF16 operand pairs (both K-contiguous): kind::f16 MMAs with
// M = 256 (the FP8 operand, widened to BF16 in shared memory) x N = 256 (the BF16 operand) per pair.
//
// STATUS: correct (its own parity matrix passes) but NOT selected by default -- on B200 it measures 1.6 times
// slower than the one-CTA mixed kernel (4096 x 4096 x 16384: 849 us against 522 us; a BF16 x BF16 problem of that
// shape takes 405 us on the FP8 / BF16 pair kernel).  Kept selectable through the MIXED_PAIR switch.
//
// Why a pair: the one-CTA mixed kernel (gemm_tc.cu) keeps a 56 KiB stage -- raw FP8 box, its widened copy and the
// BF16 box -- occupied from the moment its TMA loads are issued until its MMAs have retired, and only four such
// stages fit.  In a pair each CTA holds half of both operands: 128 rows of the FP8 operand (its own 128 TMEM lanes)
// and 128 of the pair tile's 256 BF16 rows -- 16 KiB widened + 16 KiB BF16 per k-block of 64 -- so five stages fit
// beside a ring of five 8 KiB slots for the raw FP8 boxes (freed as soon as they have been widened), and half as
// many bytes come from L2 and DRAM per FLOP.
//
// What was measured on the way (4096 x 4096 x 16384, E5M2 x BF16 -> FP32):
//   * raw ring of three slots, all eight warps widening every k-block together: 1280 us.  Too few raw loads in flight.
//   * no raw ring: the widening warps fetch their 16-byte pieces themselves, six k-blocks ahead, into registers:
//     1518 us.  Switching parts of the pass off located the cost: the release-ordered arrival on the leader's
//     barrier must wait for the thread's outstanding global loads of later k-blocks (a relaxed arrival: 1204 us;
//     no prefetch loads: 1148 us); with no stores, no proxy fence, a relaxed arrival and no loads the barrier
//     protocol alone still takes 475 us.
//   * this version -- TMA-fed raw ring of five slots (nothing outstanding in the widening threads), two groups of
//     four warps taking k-blocks in turn so that two widening passes overlap: 849 us.  What remains is the pass
//     itself: two barrier waits, shared-memory read, convert, swizzled write, proxy fence and a cluster-scope
//     release arrival per k-block, in both CTAs, before the leader may issue.
//
// Roles per CTA (11 warps): warp 0 loads the BF16 halves (both CTAs' bytes are counted on the leader's "full"
// barrier), warp 10 loads the raw FP8 boxes (local barrier), warps 2..9 widen into the MMA stage (fence towards the
// async proxy, then one arrival per warp of the group on the LEADER's "ready" barrier, remotely from the peer) and
// drain the accumulator after the tile's last k-block, warp 1 of the leader issues the MMAs once a stage is both
// full and ready and commits to both CTAs' "empty" barriers.  Two 256-column accumulators alternate.  Every wait is
// bounded; a wait that runs out raises the abort flag of both CTAs; the pair meets at a cluster barrier before
// tensor memory is released.  No load is multicast.
//
// TR = true: the caller swapped the operand roles so that the FP8 operand sits on the M side (an FP8 A): TMEM
// lanes are rows i of D, TMEM columns are columns j, m / n arrive swapped (as in the one-CTA kernel).
#pragma once
#include "gemm_tc2.cuh"

namespace e5b {
namespace tc {

constexpr int X_STAGES = 5;                                   // MMA ring
constexpr int X_RAW = 5;                                      // raw FP8 ring
constexpr int X_GROUPS = 2;                                   // groups of widening warps that take k-blocks in turn
constexpr int X_WIDE_BYTES = 128 * STAGE_K_BYTES;             // widened FP8 half: 128 rows x 64 BF16
constexpr int X_STAGE_BYTES = X_WIDE_BYTES + P_HALF_BYTES;    // + this CTA's 128 BF16 rows
constexpr int X_RAW_BYTES = 128 * (STAGE_K_BYTES / 2);        // 128 rows x 64 codes
constexpr int X_SMEM_BYTES = X_STAGES * X_STAGE_BYTES + X_RAW * X_RAW_BYTES + 1024 + 512;
constexpr int X_THREADS = THREADS + 32;

// map_f: the FP8 operand (M side), boxes of 128 rows x 64 bytes, not swizzled.  map_b / map_b2 / map_b4: the BF16
// operand (N side), boxes of 128 / 64 / 32 rows x 128 bytes, 128-byte swizzle (whole tiles, slices of the last round).
template <int DT, int FT, bool TR>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(X_THREADS, 1)
gemm_tc_mixpair_kernel(const __grid_constant__ CUtensorMap map_f, const __grid_constant__ CUtensorMap map_b,
                       const __grid_constant__ CUtensorMap map_b2, const __grid_constant__ CUtensorMap map_b4, int m, int n,
                       int k, uint32_t idesc, PairSplit ps, OutDesc o, EpiMode md) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t ring = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t *ring_p = smem_raw + (ring - smem_u32(smem_raw));
  const uint32_t rawring = ring + X_STAGES * X_STAGE_BYTES;
  uint8_t *rawring_p = ring_p + X_STAGES * X_STAGE_BYTES;
  uint64_t *bars = reinterpret_cast<uint64_t *>(rawring_p + X_RAW * X_RAW_BYTES);
  // full[S], empty[S], ready[S], raw_full[R], raw_empty[R], acc_full[2], acc_empty[2]
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 3 * X_STAGES + 2 * X_RAW + 4);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
  const uint32_t bar0 = smem_u32(bars);
  const auto full_bar = [&](int s) { return bar0 + 8u * s; };
  const auto empty_bar = [&](int s) { return bar0 + 8u * (X_STAGES + s); };
  const auto ready_bar = [&](int s) { return bar0 + 8u * (2 * X_STAGES + s); };
  const auto raw_full = [&](int r) { return bar0 + 8u * (3 * X_STAGES + r); };
  const auto raw_empty = [&](int r) { return bar0 + 8u * (3 * X_STAGES + X_RAW + r); };
  const auto acc_full = [&](int b) { return bar0 + 8u * (3 * X_STAGES + 2 * X_RAW + b); };
  const auto acc_empty = [&](int b) { return bar0 + 8u * (3 * X_STAGES + 2 * X_RAW + 2 + b); };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();
  const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
  // m: extent along the N side (BF16 operand rows, TMEM columns), n: extent along the M side (FP8 operand rows)
  const int tiles_i = (m + P_TILE - 1) / P_TILE, tiles_j = (n + P_TILE - 1) / P_TILE, tiles = tiles_i * tiles_j;
  const int kblocks = (k + 63) / 64;

  const int full_items = (tiles / pairs) * pairs, rest = tiles - full_items;
  const int f = (md.split && rest > 0) ? (4 * rest <= pairs ? 4 : (2 * rest <= pairs ? 2 : 1)) : 1;
  const int items = full_items + f * rest;
  const auto item_at = [&](int item, int &i0, int &j0, int &cols) {
    int tile = item, sub = 0;
    cols = P_TILE;
    if (item >= full_items) { const int h = item - full_items; tile = full_items + h / f; sub = h % f; cols = P_TILE / f; }
    int ti, tj;
    tile_coords(tile, tiles_i, tiles_j, ti, tj);
    i0 = ti * P_TILE + sub * cols;
    j0 = tj * P_TILE;
  };

  if (threadIdx.x == 32) { prefetch_map(&map_f); prefetch_map(&map_b); prefetch_map(&map_b2); prefetch_map(&map_b4); }
  if (threadIdx.x == 0) {
    for (int s = 0; s < X_STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); mbar_init(ready_bar(s), 2 * EPI_WARPS / X_GROUPS); }
    for (int r = 0; r < X_RAW; ++r) { mbar_init(raw_full(r), 1); mbar_init(raw_empty(r), EPI_WARPS / X_GROUPS); }
    for (int b = 0; b < 2; ++b) { mbar_init(acc_full(b), 1); mbar_init(acc_empty(b), 2 * EPI_WARPS); }
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
  const uint32_t peer_abort = map_to_rank(smem_u32(const_cast<int *>(abort_flag)), rank ^ 1u);

  if (warp == 0) {
    // ---------------- BF16 producer (both CTAs) ----------------
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int t = pair; t < items && ok; t += pairs) {
        int i0, j0, cols;
        item_at(t, i0, j0, cols);
        const int ir = i0 + (int)rank * (cols / 2);
        const CUtensorMap *mb = cols == P_TILE ? &map_b : (cols == P_TILE / 2 ? &map_b2 : &map_b4);
        const uint32_t pair_bytes = 2u * (uint32_t)(cols / 2) * STAGE_K_BYTES;
        const bool backwards = ((t / pairs) & 1) != 0;
        for (int kq = 0; kq < kblocks; ++kq) {
          const int kb = backwards ? kblocks - 1 - kq : kq;
          if (!mbar_wait(empty_bar(s), ph ^ 1u, abort_flag, (1u << 24) | (uint32_t)kb, peer_abort)) { ok = false; break; }
          if (rank == 0) mbar_expect_tx(full_bar(s), pair_bytes);
          tma_load_2d_pair(ring + s * X_STAGE_BYTES + X_WIDE_BYTES, mb, kb * 64, ir, map_to_rank(full_bar(s), 0));
          if (++s == X_STAGES) { s = 0; ph ^= 1u; }
        }
      }
    }
  } else if (warp == EPI_WARPS + 2) {
    // ---------------- raw FP8 producer (both CTAs, local ring) ----------------
    if (lane == 0) {
      int r = 0;
      uint32_t rph = 0;
      bool ok = true;
      for (int t = pair; t < items && ok; t += pairs) {
        int i0, j0, cols;
        item_at(t, i0, j0, cols);
        const int jr = j0 + (int)rank * 128;
        const bool backwards = ((t / pairs) & 1) != 0;
        for (int kq = 0; kq < kblocks; ++kq) {
          const int kb = backwards ? kblocks - 1 - kq : kq;
          if (!mbar_wait(raw_empty(r), rph ^ 1u, abort_flag, (6u << 24) | (uint32_t)kb, peer_abort)) { ok = false; break; }
          mbar_expect_tx(raw_full(r), X_RAW_BYTES);
          tma_load_2d(rawring + r * X_RAW_BYTES, &map_f, kb * 64, jr, raw_full(r));
          if (++r == X_RAW) { r = 0; rph ^= 1u; }
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
        int i0, j0, cols;
        item_at(t, i0, j0, cols);
        const uint32_t idesc_t = cols == P_TILE ? idesc : (cols == P_TILE / 2 ? ps.idesc2 : ps.idesc4);
        const uint32_t buf = lt & 1u, use = lt >> 1;
        if (!mbar_wait(acc_empty(buf), (use & 1u) ^ 1u, abort_flag, (2u << 24) | 0xFFFFu, peer_abort)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * P_TILE;
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(full_bar(s), ph, abort_flag, (2u << 24) | (uint32_t)kb, peer_abort)) { ok = false; break; }
          if (!mbar_wait(ready_bar(s), ph, abort_flag, (4u << 24) | (uint32_t)kb, peer_abort)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sw = ring + s * X_STAGE_BYTES, sb = sw + X_WIDE_BYTES;
          const uint64_t dw = kmajor_sw128_desc(sw), db = kmajor_sw128_desc(sb);
#pragma unroll
          for (int ks = 0; ks < STAGE_K_BYTES / MMA_K_BYTES; ++ks)
            mma_ss_pair<1>(d_tmem, dw + 2u * ks, db + 2u * ks, idesc_t, (kb | ks) != 0);
          mma_commit_pair(empty_bar(s));
          mma_commit_pair(map_to_rank(empty_bar(s), 1));
          if (++s == X_STAGES) { s = 0; ph ^= 1u; }
        }
        if (ok) {
          mma_commit_pair(acc_full(buf));
          mma_commit_pair(map_to_rank(acc_full(buf), 1));
        }
      }
    }
  } else {
    // ---------------- widening, then epilogue (warps 2..9 of both CTAs) ----------------
    const int quad = warp & 3, half = (warp - 2) >> 2, ct = threadIdx.x - 64;
    const OutScalars r_ = out_begin(o);
    const float as_const = __fmul_rn(o.alpha, o.sa_vec ? 1.f : ld_or_one(o.sa));
    const float sb_const = o.sb_vec ? 1.f : ld_or_one(o.sb);
    float mx = 0.f;
    uint32_t it = 0, lt = 0;     // it: k-blocks since the kernel started (ring positions); lt: tiles of this pair
    bool ok = true;
    // The eight warps form X_GROUPS groups that take k-blocks in turn: one pass over a k-block (two waits, read,
    // convert, write, proxy fence, remote arrival) is a chain of dependent latencies, and groups overlap such chains.
    constexpr int GT = 32 * EPI_WARPS / X_GROUPS;
    const int grp = ct / GT, cg = ct - grp * GT;
    for (int t = pair; t < items && ok; t += pairs, ++lt) {
      int i0, j0, cols;
      item_at(t, i0, j0, cols);
      for (int kb = 0; kb < kblocks; ++kb, ++it) {
        if ((int)(it % X_GROUPS) != grp) continue;      // warp-uniform
        const int s = it % X_STAGES, r = it % X_RAW;
        const uint32_t ph = (it / X_STAGES) & 1u, rph = (it / X_RAW) & 1u;
        ok = mbar_wait(raw_full(r), rph, abort_flag, (5u << 24) | (uint32_t)kb, peer_abort) &&
             mbar_wait(empty_bar(s), ph ^ 1u, abort_flag, (7u << 24) | (uint32_t)kb, peer_abort);
        ok = __all_sync(0xFFFFFFFFu, ok);
        if (!ok) break;
        widen_block<FT, false, GT>(rawring_p + r * X_RAW_BYTES, ring_p + s * X_STAGE_BYTES, cg);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy writes -> tensor-core reads
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(raw_empty(r));
          mbar_arrive_cluster(map_to_rank(ready_bar(s), 0));
        }
      }
      if (!ok) break;
      const uint32_t buf = lt & 1u, use = lt >> 1;
      ok = mbar_wait(acc_full(buf), use & 1u, abort_flag, (3u << 24) | (uint32_t)warp, peer_abort);
      ok = __all_sync(0xFFFFFFFFu, ok);
      if (!ok) break;
      tc_fence_after();
      const int j = j0 + (int)rank * 128 + quad * 32 + lane;     // index along the M side: column j, or row i when TR
      const bool col_ok = j < n;
      const float sbj = col_ok && o.sb_vec && !TR ? o.sb[j] : sb_const;
      float as_i = as_const, bias_i = 0.f;
      if (TR && col_ok) {
        if (o.sa_vec) as_i = __fmul_rn(o.alpha, o.sa[j]);
        if (o.bias) bias_i = load_elem(o.bias_dtype, o.bias, (size_t)j, 1.f);
      }
      const uint32_t t_lane = tmem_base + ((uint32_t)(quad * 32) << 16) + buf * P_TILE;
      for (int c0 = half * (P_TILE / 2); c0 < (half + 1) * (P_TILE / 2); c0 += 32) {
        if (c0 >= cols || i0 + c0 >= m) break;   // warp-uniform
        float acc[32];
        tmem_ld32(t_lane + c0, acc);
        if (col_ok) {
          if (TR) mx = fmaxf(mx, drain32_t<DT>(o, r_, acc, j, i0 + c0, m, as_i, sb_const, bias_i));
          else mx = fmaxf(mx, drain32<DT>(o, r_, md, acc, i0 + c0, j, m, as_const, sbj));
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_rank(acc_empty(buf), 0));
      if (!TR) {
        const int rb = i0 + half * (P_TILE / 2), re_ = i0 + (half + 1) * (P_TILE / 2);
        const int rend = re_ < i0 + cols ? re_ : i0 + cols;
        bcast_block<DT>(o, j0 + (int)rank * 128 + quad * 32, n, rb, rend < m ? rend : m);
      }
    }
    if (o.amax) {
      mx = warp_max(mx);
      if (lane == 0) amax_publish(o.amax, mx);
    }
  }

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

template <int DT, int FT, bool TR>
static cudaError_t launch_mixpair_cfg(const CUtensorMap &mf, const CUtensorMap *mb, int m, int n, int k, uint32_t idesc,
                                      const PairSplit &ps, const OutDesc &o, const EpiMode &md, int sms, cudaStream_t s) {
  static SmemOptIn optin;
  if (const cudaError_t e = optin.ensure(gemm_tc_mixpair_kernel<DT, FT, TR>, X_SMEM_BYTES)) return e;
  const int tiles = ((m + P_TILE - 1) / P_TILE) * ((n + P_TILE - 1) / P_TILE);
  int pairs = sms / 2;
  if (tiles < pairs) pairs = tiles;
  note_route(ROUTE_TC_MIXED_PAIR);
  gemm_tc_mixpair_kernel<DT, FT, TR><<<2 * pairs, X_THREADS, X_SMEM_BYTES, s>>>(mf, mb[0], mb[1], mb[2], m, n, k, idesc, ps, o, md);
  return cudaGetLastError();
}

template <int FT, bool TR>
static cudaError_t launch_mixpair_dt(const CUtensorMap &mf, const CUtensorMap *mb, int m, int n, int k, uint32_t idesc,
                                     const PairSplit &ps, const OutDesc &o, const EpiMode &md, int sms, cudaStream_t s) {
  switch (o.d_dtype) {
    case E5MA_BF16: return launch_mixpair_cfg<E5MA_BF16, FT, TR>(mf, mb, m, n, k, idesc, ps, o, md, sms, s);
    case E5MA_FP32: return launch_mixpair_cfg<E5MA_FP32, FT, TR>(mf, mb, m, n, k, idesc, ps, o, md, sms, s);
    case E5MA_FP16: return launch_mixpair_cfg<E5MA_FP16, FT, TR>(mf, mb, m, n, k, idesc, ps, o, md, sms, s);
    case E5MA_E5M2: return launch_mixpair_cfg<E5MA_E5M2, FT, TR>(mf, mb, m, n, k, idesc, ps, o, md, sms, s);
    default: return launch_mixpair_cfg<E5MA_E4M3, FT, TR>(mf, mb, m, n, k, idesc, ps, o, md, sms, s);
  }
}

}  // namespace tc
}  // namespace e5b
