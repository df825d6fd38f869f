// Tensor-core GEMM on CTA pairs (tcgen05 cta_group::2): two CTAs of a 2-CTA cluster compute one
// 256 (columns j) x 256 (rows i) output tile together.  Used for large FP8 x FP8 and BF16 x BF16
// problems with both operands K-contiguous; smaller or mixed problems take the one-CTA kernel.
//
// Why pairs: the one-CTA kernel moves 48 KiB of operands from L2 into shared memory per
// 128 x 256 x 128-byte k-block; with every SM doing that the L2-to-SM traffic (and the power it
// costs on a power-capped part) is what limits it.  In a pair each CTA loads only its own half of
// both operands -- 128 rows of op(B)^T and 128 rows of op(A), 32 KiB per k-block -- and the MMA unit
// reads the other half from the peer's shared memory.  No load is multicast: every byte is fetched
// by exactly one of the two CTAs, for itself.
//
// Roles per CTA (10 warps, as in the one-CTA kernel):
//   warp 0  TMA producer.  Both CTAs load their halves; the transaction bytes of both are counted on
//           the leader's (cluster rank 0) "full" barrier, which the leader arms for the whole pair.
//   warp 1  MMA issuer, active in the leader only: M = 256 (128 TMEM lanes in each CTA), N = 256.
//           After a k-block it commits to the "empty" barrier of both CTAs (two commits, one per
//           barrier), after the last one to both CTAs' "accumulator full" barriers.
//   warps 2..9  epilogue: each CTA drains its own 128 TMEM lanes (its 128 columns j) exactly as in the
//           one-CTA kernel, then arrives on the leader's "accumulator empty" barrier (remotely
//           from the peer).
// Every wait is bounded as in the one-CTA kernel; before releasing tensor memory and exiting the
// two CTAs meet at a cluster barrier, so neither leaves while the other may still touch its
// shared memory.
#pragma once
#include "tc_common.cuh"

namespace e5b {
namespace tc {

constexpr int P_STAGES = 6;
constexpr int P_HALF_BYTES = 128 * STAGE_K_BYTES;        // one operand half: 128 rows x 128 bytes
constexpr int P_STAGE_BYTES = 2 * P_HALF_BYTES;          // this CTA's halves of both operands
constexpr int P_SMEM_BYTES = P_STAGES * P_STAGE_BYTES + 1024 + 384;
constexpr int P_TILE = 256;

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// address of the same shared-memory location in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_rank(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA load whose completion bytes are counted on a barrier that may live in the peer CTA
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap *map, int c0, int c1, uint32_t bar_cluster) {
  asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
               ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar_cluster) : "memory");
}
template <int KIND>
__device__ __forceinline__ void mma_ss_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  if (KIND == 0)
    asm volatile("{ .reg .pred p; setp.ne.b32 p, %4, 0; tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p; }"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
  else
    asm volatile("{ .reg .pred p; setp.ne.b32 p, %4, 0; tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p; }"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// one arrival on the given barrier (any CTA of the pair) once all MMAs issued so far have completed
__device__ __forceinline__ void mma_commit_pair(uint32_t bar_cluster) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster) : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t slot_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_smem), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}

// What the kernel needs to cut the tiles of the last, partly filled round into 2 or 4 slices along
// i: MMA N = 256 / f, boxes of 128 / f rows of op(A) per CTA.
struct PairSplit { uint32_t idesc2, idesc4; };

// map_i / map_j: tensor maps of op(A) / op(B)^T with boxes of 128 rows x 128 bytes of K;
// map_i2 / map_i4: op(A) with boxes of 64 / 32 rows (sliced tiles of the last round).
template <int KIND, int DT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_i, const __grid_constant__ CUtensorMap map_j,
                    const __grid_constant__ CUtensorMap map_i2, const __grid_constant__ CUtensorMap map_i4, int m, int n,
                    int k_bytes, uint32_t idesc, PairSplit ps, OutDesc o, EpiMode md) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t ring = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t *after_ring = smem_raw + (ring - smem_u32(smem_raw)) + P_STAGES * P_STAGE_BYTES;
  uint64_t *bars = reinterpret_cast<uint64_t *>(after_ring);   // full[S], empty[S], acc_full[2], acc_empty[2]
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * P_STAGES + 4);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
  const uint32_t bar0 = smem_u32(bars);
  const auto full_bar = [&](int s) { return bar0 + 8u * s; };
  const auto empty_bar = [&](int s) { return bar0 + 8u * (P_STAGES + s); };
  const auto acc_full = [&](int b) { return bar0 + 8u * (2 * P_STAGES + b); };
  const auto acc_empty = [&](int b) { return bar0 + 8u * (2 * P_STAGES + 2 + b); };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();          // 0: leader (issues the MMAs), 1: peer
  const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
  const int tiles_i = (m + P_TILE - 1) / P_TILE, tiles_j = (n + P_TILE - 1) / P_TILE, tiles = tiles_i * tiles_j;
  const int kblocks = (k_bytes + STAGE_K_BYTES - 1) / STAGE_K_BYTES;

  // Work items: tiles dealt round-robin to the pairs.  When the last round would leave most pairs idle,
  // its tiles are cut into f = 2 or 4 slices of 256 / f rows i (the largest f with f * rest <= pairs), so
  // that the round takes 1 / f of the time.  Every role of both CTAs derives the same list.
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

  if (threadIdx.x == 32) { prefetch_map(&map_i); prefetch_map(&map_j); prefetch_map(&map_i2); prefetch_map(&map_i4); }
  if (threadIdx.x == 0) {
    for (int s = 0; s < P_STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(acc_full(b), 1); mbar_init(acc_empty(b), 2 * EPI_WARPS); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {   // the same warp of both CTAs takes part in the paired allocation
    tmem_alloc_pair(smem_u32(tmem_slot), 512);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();          // both CTAs' barriers are initialised before anyone signals the other
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t peer_abort = map_to_rank(smem_u32(const_cast<int *>(abort_flag)), rank ^ 1u);   // the other CTA's abort flag

  if (warp == 0) {
    // ---------------- TMA producer (both CTAs) ----------------
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int t = pair; t < items && ok; t += pairs) {
        int i0, j0, cols;
        item_at(t, i0, j0, cols);
        i0 += (int)rank * (cols / 2);     // this CTA's half of the N side
        j0 += (int)rank * 128;            // and its 128 rows of the M side
        const CUtensorMap *mi = cols == P_TILE ? &map_i : (cols == P_TILE / 2 ? &map_i2 : &map_i4);
        const uint32_t pair_bytes = 2u * (P_HALF_BYTES + (uint32_t)(cols / 2) * STAGE_K_BYTES);
        // Successive tiles of a pair walk K in opposite directions: the next tile starts with the k-blocks its
        // predecessors in the same band read last, which are the ones still in L2 (the sum does not care
        // about the order of its k-blocks).
        const bool backwards = ((t / pairs) & 1) != 0;
        for (int kq = 0; kq < kblocks; ++kq, ++it) {
          const int kb = backwards ? kblocks - 1 - kq : kq;
          const int s = it % P_STAGES;
          const uint32_t ph = (it / P_STAGES) & 1u;
          if (!mbar_wait(empty_bar(s), ph ^ 1u, abort_flag, (1u << 24) | (uint32_t)kb, peer_abort)) { ok = false; break; }
          const uint32_t lead_full = map_to_rank(full_bar(s), 0);
          if (rank == 0) mbar_expect_tx(full_bar(s), pair_bytes);   // both CTAs' bytes land on this barrier
          const uint32_t sj = ring + s * P_STAGE_BYTES, si = sj + P_HALF_BYTES;
          const int kc = kb * (KIND == 0 ? STAGE_K_BYTES : STAGE_K_BYTES / 2);
          tma_load_2d_pair(sj, &map_j, kc, j0, lead_full);
          tma_load_2d_pair(si, mi, kc, i0, lead_full);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (leader CTA only) ----------------
    if (lane == 0 && rank == 0) {
      uint32_t it = 0, lt = 0;
      bool ok = true;
      for (int t = pair; t < items && ok; t += pairs, ++lt) {
        int i0, j0, cols;
        item_at(t, i0, j0, cols);
        const uint32_t idesc_t = cols == P_TILE ? idesc : (cols == P_TILE / 2 ? ps.idesc2 : ps.idesc4);
        const uint32_t buf = lt & 1u, use = lt >> 1;
        if (!mbar_wait(acc_empty(buf), (use & 1u) ^ 1u, abort_flag, (2u << 24) | 0xFFFFu, peer_abort)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * P_TILE;
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const int s = it % P_STAGES;
          const uint32_t ph = (it / P_STAGES) & 1u;
          if (!mbar_wait(full_bar(s), ph, abort_flag, (2u << 24) | (uint32_t)kb, peer_abort)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sj = ring + s * P_STAGE_BYTES, si = sj + P_HALF_BYTES;
          const uint64_t dj = kmajor_sw128_desc(sj), di = kmajor_sw128_desc(si);
#pragma unroll
          for (int ks = 0; ks < STAGE_K_BYTES / MMA_K_BYTES; ++ks)
            mma_ss_pair<KIND>(d_tmem, dj + 2u * ks, di + 2u * ks, idesc_t, (kb | ks) != 0);
          mma_commit_pair(empty_bar(s));                   // this CTA's stage is free again
          mma_commit_pair(map_to_rank(empty_bar(s), 1));   // and the peer's
        }
        if (ok) {
          mma_commit_pair(acc_full(buf));
          mma_commit_pair(map_to_rank(acc_full(buf), 1));
        }
      }
    }
  } else {
    // ---------------- epilogue (both CTAs): own 128 TMEM lanes = columns j0 + rank * 128 ... ----------------
    const int quad = warp & 3, half = (warp - 2) >> 2;
    const OutScalars r = out_begin(o);
    const float as_const = __fmul_rn(o.alpha, o.sa_vec ? 1.f : ld_or_one(o.sa));
    const float sb_const = o.sb_vec ? 1.f : ld_or_one(o.sb);
    float mx = 0.f;
    uint32_t lt = 0;
    bool ok = true;
    for (int t = pair; t < items && ok; t += pairs, ++lt) {
      int i0, j0, cols;
      item_at(t, i0, j0, cols);
      j0 += (int)rank * 128;
      const uint32_t buf = lt & 1u, use = lt >> 1;
      ok = mbar_wait(acc_full(buf), use & 1u, abort_flag, (3u << 24) | (uint32_t)warp, peer_abort);
      ok = __all_sync(0xFFFFFFFFu, ok);
      if (!ok) break;
      tc_fence_after();
      const int j = j0 + quad * 32 + lane;
      const bool col_ok = j < n;
      const float sbj = col_ok && o.sb_vec ? o.sb[j] : sb_const;
      const uint32_t t_lane = tmem_base + ((uint32_t)(quad * 32) << 16) + buf * P_TILE;
      for (int c0 = half * (P_TILE / 2); c0 < (half + 1) * (P_TILE / 2); c0 += 32) {
        if (c0 >= cols || i0 + c0 >= m) break;   // warp-uniform
        float acc[32];
        tmem_ld32(t_lane + c0, acc);
        if (col_ok) mx = fmaxf(mx, drain32<DT>(o, r, md, acc, i0 + c0, j, m, as_const, sbj));
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_rank(acc_empty(buf), 0));
      // e5b_gemm_bcast: this warp's block of the tile goes to the peers while the MMA warp is already filling the buffer again
      const int rb = i0 + half * (P_TILE / 2), re_ = i0 + (half + 1) * (P_TILE / 2);
      const int rend = re_ < i0 + cols ? re_ : i0 + cols;
      bcast_block<DT>(o, j0 + quad * 32, n, rb, rend < m ? rend : m);
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

template <int KIND, int DT>
static cudaError_t launch_pair_cfg(const CUtensorMap &mi, const CUtensorMap &mj, const CUtensorMap &mi2, const CUtensorMap &mi4,
                                   int m, int n, int k_bytes, uint32_t idesc, const PairSplit &ps, const OutDesc &o,
                                   const EpiMode &md, int sms, cudaStream_t s) {
  static SmemOptIn optin;
  if (const cudaError_t e = optin.ensure(gemm_tc_pair_kernel<KIND, DT>, P_SMEM_BYTES)) return e;
  note_route(ROUTE_TC_PAIR);
  const int tiles = ((m + P_TILE - 1) / P_TILE) * ((n + P_TILE - 1) / P_TILE);
  int pairs = sms / 2;
  if (tiles < pairs) pairs = tiles;
  gemm_tc_pair_kernel<KIND, DT><<<2 * pairs, THREADS, P_SMEM_BYTES, s>>>(mi, mj, mi2, mi4, m, n, k_bytes, idesc, ps, o, md);
  return cudaGetLastError();
}

template <int KIND>
static cudaError_t launch_pair(const CUtensorMap &mi, const CUtensorMap &mj, const CUtensorMap &mi2, const CUtensorMap &mi4,
                               int m, int n, int k_bytes, uint32_t idesc, const PairSplit &ps, const OutDesc &o,
                               const EpiMode &md, int sms, cudaStream_t s) {
  switch (o.d_dtype) {
    case E5MA_BF16: return launch_pair_cfg<KIND, E5MA_BF16>(mi, mj, mi2, mi4, m, n, k_bytes, idesc, ps, o, md, sms, s);
    case E5MA_FP32: return launch_pair_cfg<KIND, E5MA_FP32>(mi, mj, mi2, mi4, m, n, k_bytes, idesc, ps, o, md, sms, s);
    case E5MA_FP16: return launch_pair_cfg<KIND, E5MA_FP16>(mi, mj, mi2, mi4, m, n, k_bytes, idesc, ps, o, md, sms, s);
    case E5MA_E5M2: return launch_pair_cfg<KIND, E5MA_E5M2>(mi, mj, mi2, mi4, m, n, k_bytes, idesc, ps, o, md, sms, s);
    default: return launch_pair_cfg<KIND, E5MA_E4M3>(mi, mj, mi2, mi4, m, n, k_bytes, idesc, ps, o, md, sms, s);
  }
}

}  // namespace tc
}  // namespace e5b
