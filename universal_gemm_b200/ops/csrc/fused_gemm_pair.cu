// Fused stationary GEMM, CTA-pair variant (tcgen05 cta_group::2) for sm_100a.
//
// Same tables, roles and fetch / remote-accumulate protocol as fused_gemm.cu, but two CTAs of a
// cluster (two SMs) compute one 256 x 256 output tile together:
//   * each CTA loads 128 rows of A and 128 of the 256 B columns per K block (32 KiB; a stage holds two K blocks,
//     3 stages of 64 KiB), so an SM needs 64 operand bytes per tensor cycle, like the one-CTA 256-row tile;
//   * each CTA's TMEM holds its 128 rows x 256 columns, i.e. only half of TMEM, so the accumulators are
//     double buffered and the epilogue (which may push over NVLink) hides behind the next main loop,
//     like the one-CTA 128-row tile.
// A second instantiation (kWide) computes 256 x 512 tiles: each CTA loads 128 rows of A and 2 x 128 columns of B
// per K block (48 KiB per stage, 4 stages), so an SM needs 48 operand bytes per tensor cycle and every byte in
// flight feeds twice the tensor time; its 128 x 512 accumulators fill TMEM, so the epilogue is not hidden.
// CTA rank 0 of the pair issues the UMMAs; TMA loads of both CTAs complete on rank 0's "full" barrier
// (cp.async.bulk.tensor with .cta_group::2, never multicast); UMMA completion is committed to the
// "empty" / "accumulator full" barriers of both CTAs with two plain commits.  With dynamic tile claiming the leader's
// producer claims tiles and writes them into both CTAs' tile queues (a plain 64-bit store into the other CTA's
// shared memory).
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <string.h>

#include "fused_common.cuh"

using namespace ugptx;
using namespace ugfused;

namespace {

constexpr int kPairStages = 6;                                  // most stages of any instantiation
constexpr uint32_t kPairABytes = 128 * UG_BK * 2;               // 16 KiB: this CTA's 128 rows of A
constexpr uint32_t kPairHalfBBytes = 2 * kBChunkBytes;          // 16 KiB: this CTA's 128 columns of one 256-column UMMA
constexpr uint32_t kPairRingBytes = 6 * (kPairABytes + kPairHalfBBytes);   // 192 KiB = 4 x 48 KiB as well
constexpr uint32_t kPairSmemBytes = kPairRingBytes + 1024 + kCtlBytes + kEpiBytes;

template <bool kWide>
struct PairCfg {
  // A stage holds kKps K blocks (sub-stages); one full / empty barrier round trip and one pair of commits per stage.
  // The 256-column tile takes two K blocks per stage: with one, the per-stage work of the issuing thread (barrier
  // wait, fence, four UMMAs, two commits) took longer than the 512 tensor cycles the stage feeds.
  static constexpr int kKps = kWide ? 1 : 2;
  static constexpr uint32_t kSubBytes = kPairABytes + (kWide ? 2u : 1u) * kPairHalfBBytes;   // 48 / 32 KiB per K block
  static constexpr uint32_t kStageBytes = kKps * kSubBytes;                                   // 48 / 64 KiB
  static constexpr int kStages = kWide ? 4 : 3;
  static constexpr int kAccBufs = kWide ? 1 : 2;
  static_assert(kStages * kStageBytes == kPairRingBytes, "ring size");
};

struct PairShared {
  uint64_t full[kPairStages];     // used in rank 0: bytes of both CTAs' loads
  uint64_t empty[kPairStages];    // per CTA: stage consumed by the pair UMMAs
  uint64_t acc_full[2];           // per CTA: accumulator buffer complete
  uint64_t acc_empty[2];          // used in rank 0: both CTAs' epilogues drained the buffer
  uint32_t tmem_base;
  volatile uint32_t abort;
  TileQueue tq;                   // per CTA; the leader's producer writes both CTAs' queues
};
static_assert(sizeof(PairShared) <= kCtlBytes, "control block overlaps the epilogue buffers");

// Instruction descriptor of the pair UMMA: M = 256 (128 per CTA), N = n (256, or 128 for tail tiles).
__device__ __forceinline__ uint32_t make_idesc_pair(uint32_t n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (0u << 15) | (1u << 16) | ((n >> 3) << 17) | ((256u >> 4) << 24);
}

template <bool kWide>
__global__ void __launch_bounds__(kNumThreads, 1) ug_fused_gemm_pair_kernel(const UgFusedParams P) {
  using C = PairCfg<kWide>;
  constexpr int kStages = C::kStages;
  constexpr int kKps = C::kKps;
  constexpr uint32_t kStageBytes = C::kStageBytes;
  constexpr uint32_t kSubBytes = C::kSubBytes;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t ring = (raw_addr + 1023u) & ~1023u;
  PairShared* sh = reinterpret_cast<PairShared*>(smem_raw + (ring - raw_addr) + kPairRingBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();          // 0 = leader of the pair
  const int pair_id = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  const UgTask* __restrict__ tasks = reinterpret_cast<const UgTask*>(P.tasks);
  const UgSegment* __restrict__ segs = reinterpret_cast<const UgSegment*>(P.segs);
  const uint32_t* flags = reinterpret_cast<const uint32_t*>(P.flags);
  const int32_t* __restrict__ flag_need = reinterpret_cast<const int32_t*>(P.flag_need);

  WaitCtl ctl;
  ctl.abort = &sh->abort;
  ctl.status = reinterpret_cast<uint32_t*>(P.status);
  ctl.deadline = global_timer_ns() + P.timeout_ns;
  ctl.peer_abort = mapa_shared(smem_u32(const_cast<uint32_t*>(&sh->abort)), rank ^ 1u);
  // Static schedule: pair p runs tiles p, p + pairs, ...  Dynamic: after its first tile the leader CTA's producer
  // claims the next unclaimed tile from a global counter and writes it into the tile queues of both CTAs.
  const bool dyn = P.sched != 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kPairStages; ++s) {
      mbar_init(smem_u32(&sh->full[s]), 1);
      mbar_init(smem_u32(&sh->empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&sh->acc_full[b]), 1);
      mbar_init(smem_u32(&sh->acc_empty[b]), 2 * kNumEpiWarps * 32);
    }
    sh->abort = 0;
    for (int i = 0; i < kTileQueueSlots; ++i) sh->tq.slot[i] = 0ull;
    fence_mbar_init();
    if (uint64_t* ts = trace_summary(P, blockIdx.x)) {
      ts[UG_TR_S_START] = global_timer_ns();
      ts[UG_TR_S_CLK_START] = static_cast<uint64_t>(clock64());
    }
  }
  if (warp == kMmaWarp) {
    tmem_alloc_pair(smem_u32(&sh->tmem_base), kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();              // barriers of both CTAs are initialised before anyone signals them
  tc_fence_after();
  const uint32_t tmem_base = sh->tmem_base;

  if (warp == kProducerWarp) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      uint64_t seen[4] = {0, 0, 0, 0};
      bool ok = true;
      int tile = pair_id;
      for (int iter = 0; ok; ++iter) {
        if (!dyn) {
          if (iter > 0) tile += num_pairs;
        } else if (rank == 0) {
          if (iter > 0) tile = num_pairs + static_cast<int>(atomicAdd(reinterpret_cast<uint32_t*>(P.sched), 1u));
          const uint32_t slot = smem_u32(const_cast<unsigned long long*>(&sh->tq.slot[iter & (kTileQueueSlots - 1)]));
          st_shared_cluster_u64(mapa_shared(slot, 1), tileq_word(iter, tile));   // the other CTA's queue
          tileq_publish(&sh->tq, iter, tile);
        } else {
          tile = tileq_get(&sh->tq, iter, ctl);
          if (tile < 0) break;
        }
        if (tile >= P.total_tiles) break;
        const TileCoord tc = locate(tasks, P.num_tasks, tile);
        const UgTask& t = tasks[tc.task];
        if (!task_in_bounds(P, t)) { raise_error(ctl, UG_ERR_BAD_TABLE); break; }
        // Tile width 512 (wide kernel only), 256, or 128 for tail tiles.  A tile is 1 or 2 UMMA halves of up to 256
        // columns; of each half this CTA loads its own 128 (64) columns.
        const int tile_n = task_tile_n(t);
        const int n_rem = min(tile_n, t.n - tc.nt * tile_n);
        const int halves = (kWide && n_rem > 256) ? 2 : 1;
        const int half_cols = min(tile_n, 256) >> 1;     // this CTA's columns per half
        trace_put(P, blockIdx.x, iter, UG_TR_TILE, static_cast<uint64_t>(tile) + 1u);
        trace_now(P, blockIdx.x, iter, UG_TR_PROD_BEGIN);
        uint64_t waited = 0;
        for (int s = 0; ok && s < t.seg_count; ++s) {
          const UgSegment& sg = segs[t.seg_begin + s];
          if (!segment_in_bounds(P, sg, sg.a_flag + tc.mt, sg.b_flag + (tc.nt * tile_n) / UG_BN + halves - 1)) {
            raise_error(ctl, UG_ERR_BAD_TABLE);
            ok = false;
            break;
          }
          const uint64_t w0 = (P.trace != 0 && (sg.a_flag >= 0 || sg.b_flag >= 0)) ? global_timer_ns() : 0;
          if (sg.a_flag >= 0) {
            const int f = sg.a_flag + tc.mt;
            ok = flag_wait(flags + f, static_cast<uint32_t>(flag_need[f]), ctl);
          }
          if (ok && sg.b_flag >= 0) {
            const int f = sg.b_flag + (tc.nt * tile_n) / UG_BN;
            for (int h = 0; ok && h < halves; ++h)         // a 512-column tile spans two staged chunks of 256
              ok = flag_wait(flags + f + h, static_cast<uint32_t>(flag_need[f + h]), ctl);
          }
          if (!ok) break;
          if (w0 != 0) waited += global_timer_ns() - w0;
          if (sg.a_flag >= 0 || sg.b_flag >= 0) fence_proxy_async();
          const uint64_t amap = P.maps + static_cast<uint64_t>(sg.a_map) * 128u;
          const uint64_t bmap = P.maps + static_cast<uint64_t>(sg.b_map) * 128u;
          if (sg.a_map >= 256 || !((seen[sg.a_map >> 6] >> (sg.a_map & 63)) & 1ull)) {
            tensormap_acquire(amap);
            if (sg.a_map < 256) seen[sg.a_map >> 6] |= 1ull << (sg.a_map & 63);
          }
          if (sg.b_map >= 256 || !((seen[sg.b_map >> 6] >> (sg.b_map & 63)) & 1ull)) {
            tensormap_acquire(bmap);
            if (sg.b_map < 256) seen[sg.b_map >> 6] |= 1ull << (sg.b_map & 63);
          }
          const int nkb = (sg.k_len + UG_BK - 1) / UG_BK;
          const int ay = sg.a_row0 + tc.mt * 256 + static_cast<int>(rank) * 128;
          const int bx = sg.b_col0 + tc.nt * tile_n + static_cast<int>(rank) * half_cols;
          const int chunks = half_cols > 64 ? 2 : 1;       // 64-column boxes per half
          const uint32_t cta_bytes = kPairABytes + static_cast<uint32_t>(halves * chunks) * kBChunkBytes;
          for (int kb = 0; kb < nkb; kb += kKps) {
            const int cnt = min(kKps, nkb - kb);           // K blocks in this stage
            ok = mbar_wait(smem_u32(&sh->empty[stage]), phase ^ 1u, ctl);
            if (!ok) break;
            const uint32_t full_local = smem_u32(&sh->full[stage]);
            const uint32_t full_leader = mapa_shared(full_local, 0);
            if (rank == 0) mbar_arrive_expect_tx(full_local, 2 * cta_bytes * static_cast<uint32_t>(cnt));
            for (int sub = 0; sub < cnt; ++sub) {
              const uint32_t sa = ring + stage * kStageBytes + sub * kSubBytes;
              const uint32_t sb = sa + kPairABytes;
              const int kx = (kb + sub) * UG_BK;
              tma_load_2d_pair(sa, amap, sg.a_col0 + kx, ay, full_leader);
              for (int h = 0; h < halves; ++h)
                for (int c = 0; c < chunks; ++c)
                  tma_load_2d_pair(sb + h * kPairHalfBBytes + c * kBChunkBytes, bmap, bx + h * 256 + c * 64,
                                   sg.b_row0 + kx, full_leader);
            }
            if (++stage == kStages) { stage = 0; phase ^= 1u; }
          }
        }
        trace_put(P, blockIdx.x, iter, UG_TR_PROD_FLAGWAIT, waited);
        trace_now(P, blockIdx.x, iter, UG_TR_PROD_END);
      }
    }
  } else if (warp == kMmaWarp) {
    // ------------------------------------------------------------ UMMA issuer (leader CTA only)
    if (lane == 0 && rank == 0) {
      uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
      bool ok = true;
      for (int iter = 0; ok; ++iter) {
        const int tile = dyn ? tileq_get(&sh->tq, iter, ctl) : pair_id + iter * num_pairs;
        if (tile < 0 || tile >= P.total_tiles) break;
        const TileCoord tc = locate(tasks, P.num_tasks, tile);
        const UgTask& t = tasks[tc.task];
        if (!task_in_bounds(P, t)) { raise_error(ctl, UG_ERR_BAD_TABLE); break; }   // this role reads segs[] too
        const int tile_n = task_tile_n(t);
        const int halves = (kWide && min(tile_n, t.n - tc.nt * tile_n) > 256) ? 2 : 1;
        const uint32_t idesc = make_idesc_pair(static_cast<uint32_t>(min(tile_n, 256)));
        ok = mbar_wait(smem_u32(&sh->acc_empty[acc]), acc_phase ^ 1u, ctl);
        if (!ok) break;
        tc_fence_after();
        trace_now(P, blockIdx.x, iter, UG_TR_MMA_BEGIN);
        trace_put(P, blockIdx.x, iter, UG_TR_MMA_CLK, static_cast<uint64_t>(clock64()));
        const uint32_t d_tmem = tmem_base + (C::kAccBufs == 2 ? acc * UG_BN : 0u);
        bool first = true;                                 // the first UMMA of a tile overwrites the accumulator
        for (int sgi = 0; ok && sgi < t.seg_count; ++sgi) {
          const int nkb = (segs[t.seg_begin + sgi].k_len + UG_BK - 1) / UG_BK;
          for (int kb = 0; kb < nkb; kb += kKps) {
            const int cnt = min(kKps, nkb - kb);
            ok = mbar_wait(smem_u32(&sh->full[stage]), phase, ctl);
            if (!ok) break;
            tc_fence_after();
            for (int sub = 0; sub < cnt; ++sub) {
              const uint32_t sa = ring + stage * kStageBytes + sub * kSubBytes;
              const uint32_t sb = sa + kPairABytes;
#pragma unroll
              for (int ks = 0; ks < UG_BK / 16; ++ks) {
                const uint64_t ad = make_desc_a(sa + ks * 32);
                const uint32_t accum = first ? 0u : 1u;
                first = false;
                umma_bf16_pair(d_tmem, ad, make_desc_b(sb + ks * 2048), idesc, accum);
                if (kWide && halves == 2)
                  umma_bf16_pair(d_tmem + UG_BN, ad, make_desc_b(sb + kPairHalfBBytes + ks * 2048), idesc, accum);
              }
            }
            const uint32_t e = smem_u32(&sh->empty[stage]);
            umma_commit_pair(mapa_shared(e, 0));
            umma_commit_pair(mapa_shared(e, 1));
            if (++stage == kStages) { stage = 0; phase ^= 1u; }
          }
        }
        if (!ok) break;
        const uint32_t f = smem_u32(&sh->acc_full[acc]);
        umma_commit_pair(mapa_shared(f, 0));
        umma_commit_pair(mapa_shared(f, 1));
        trace_now(P, blockIdx.x, iter, UG_TR_MMA_ISSUED);
        if (C::kAccBufs == 2) acc ^= 1u;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
  } else if (warp < kFetchWarp0) {
    // ------------------------------------------------------------ epilogue (both CTAs, own 128 rows)
    const int quad = warp & 3;                       // TMEM lane quadrant this warp may read
    const int part = (warp - kEpiWarp0) >> 2;        // 0: left part of the tile's columns, 1: right part
    const bool tracer = warp == kEpiWarp0 && lane == 0;
    float* epi_buf = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(sh) + kCtlBytes) + (warp - kEpiWarp0) * (kEpiWarpBytes / 4);
    uint32_t acc = 0, acc_phase = 0;
    bool ok = true;
    for (int iter = 0; ok; ++iter) {
      const int tile = dyn ? tileq_get(&sh->tq, iter, ctl) : pair_id + iter * num_pairs;
      if (tile < 0 || tile >= P.total_tiles) break;
      const TileCoord tc = locate(tasks, P.num_tasks, tile);
      const UgTask& t = tasks[tc.task];
      ok = mbar_wait_backoff(smem_u32(&sh->acc_full[acc]), acc_phase, ctl, static_cast<uint32_t>(P.epi_poll_ns));
      if (!ok) break;
      tc_fence_after();
      if (tracer) {
        trace_now(P, blockIdx.x, iter, UG_TR_EPI_BEGIN);
        trace_put(P, blockIdx.x, iter, UG_TR_EPI_CLK, static_cast<uint64_t>(clock64()));
      }
      const int col0 = tc.nt * task_tile_n(t);
      const int n_rem = min(task_tile_n(t), t.n - col0);
      const int row0 = tc.mt * 256 + static_cast<int>(rank) * 128 + quad * 32;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + (C::kAccBufs == 2 ? acc * UG_BN : 0u);
      // the two warps of a quadrant split the columns on a multiple of 64 (whole 128-byte row segments each)
      const int split = min(n_rem, ((n_rem + 127) >> 7) << 6);
      const int c0 = part == 0 ? 0 : split, cn = part == 0 ? split : n_rem - split;
      float csum = 0.f;
      if (row0 < t.m && cn > 0)
        epilogue_drain(taddr + c0, t, row0, col0 + c0, cn, (kWide ? 2 * UG_BN : UG_BN) - c0, epi_buf, lane,
                       P.checksum != 0 ? &csum : nullptr);
      if (tracer) trace_now(P, blockIdx.x, iter, UG_TR_EPI_END);
      tc_fence_before();
      mbar_arrive_cluster(mapa_shared(smem_u32(&sh->acc_empty[acc]), 0));
      checksum_flush(P.checksum, csum, lane);
      if (C::kAccBufs == 2) acc ^= 1u;
      if (acc == 0) acc_phase ^= 1u;
    }
  } else {
    // ------------------------------------------------------------ fetch warps
    const UgPiece* __restrict__ pieces = reinterpret_cast<const UgPiece*>(P.pieces);
    uint32_t* counter = reinterpret_cast<uint32_t*>(P.piece_counter);
    uint32_t* wflags = reinterpret_cast<uint32_t*>(P.flags);
    unsigned long long copied = 0;
    while (P.num_pieces > 0) {
      uint32_t p = 0;
      if (lane == 0) p = atomicAdd(counter, 1u);
      p = __shfl_sync(0xffffffffu, p, 0);
      if (p >= static_cast<uint32_t>(P.num_pieces) || sh->abort) break;
      const UgPiece pc = pieces[p];
      if (pc.flag < 0 || pc.flag >= P.num_flags) {      // warp-uniform: never copy for a counter that does not exist
        if (lane == 0) raise_error(ctl, UG_ERR_BAD_TABLE);
        break;
      }
      copy_piece(pc, lane, P.fetch_depth == 0 ? 16 : P.fetch_depth);
      __threadfence();
      __syncwarp();
      if (lane == 0) {
        __threadfence();
        red_release_gpu_add(wflags + pc.flag, 1u);
      }
      ++copied;
    }
    if (lane == 0 && P.num_pieces > 0) {
      if (uint64_t* ts = trace_summary(P, blockIdx.x)) {
        atomicMax(reinterpret_cast<unsigned long long*>(ts + UG_TR_S_FETCH_END),
                  static_cast<unsigned long long>(global_timer_ns()));
        atomicAdd(reinterpret_cast<unsigned long long*>(ts + UG_TR_S_PIECES), copied);
      }
    }
  }

  // ------------------------------------------------------------ teardown
  if (sh->abort) {
    const uint64_t until = global_timer_ns() + 200000ull;
    while (global_timer_ns() < until) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();              // neither CTA leaves while the other may still touch its shared memory
  tc_fence_after();
  if (warp == kMmaWarp) tmem_dealloc_pair(tmem_base, kTmemCols);
  if (threadIdx.x == 0 && dyn && rank == 0) {
    // Both CTAs of this pair are done (cluster barrier above), so the pair claims no more tiles: the last pair to
    // get here re-arms the counters for the next launch.
    uint32_t* sched = reinterpret_cast<uint32_t*>(P.sched);
    if (atomicAdd(sched + 1, 1u) == static_cast<uint32_t>(num_pairs - 1)) {
      sched[0] = 0u;
      sched[1] = 0u;
      __threadfence();
    }
  }
  if (threadIdx.x == 0) {
    if (uint64_t* ts = trace_summary(P, blockIdx.x)) {
      ts[UG_TR_S_END] = global_timer_ns();
      ts[UG_TR_S_CLK_END] = static_cast<uint64_t>(clock64());
    }
  }
}

}  // namespace

extern "C" int ug_fused_gemm_pair(const UgFusedParams* params, int grid, void* stream) {
  static bool configured[64] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (grid <= 0 || (grid & 1)) return static_cast<int>(cudaErrorInvalidValue);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    e = cudaFuncSetAttribute(ug_fused_gemm_pair_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(kPairSmemBytes));
    if (e != cudaSuccess) return static_cast<int>(e);
    e = cudaFuncSetAttribute(ug_fused_gemm_pair_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(kPairSmemBytes));
    if (e != cudaSuccess) return static_cast<int>(e);
    configured[dev] = true;
  }
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(static_cast<unsigned>(grid), 1, 1);
  cfg.blockDim = dim3(kNumThreads, 1, 1);
  cfg.dynamicSmemBytes = kPairSmemBytes;
  cfg.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  // cta_pair == 2: tables were lowered for 256 x 512 tiles (single accumulator buffer, 4 stages of 48 KiB)
  e = params->cta_pair == 2 ? cudaLaunchKernelEx(&cfg, ug_fused_gemm_pair_kernel<true>, *params)
                            : cudaLaunchKernelEx(&cfg, ug_fused_gemm_pair_kernel<false>, *params);
  return static_cast<int>(e);
}

// Largest number of CTA pairs that can be resident at once on the current device (0 on error).
extern "C" int ug_fused_gemm_pair_max_pairs(void) {
  cudaError_t e = cudaFuncSetAttribute(ug_fused_gemm_pair_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(kPairSmemBytes));
  if (e != cudaSuccess) return 0;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(2, 1, 1);
  cfg.blockDim = dim3(kNumThreads, 1, 1);
  cfg.dynamicSmemBytes = kPairSmemBytes;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  e = cudaOccupancyMaxActiveClusters(&n, ug_fused_gemm_pair_kernel<false>, &cfg);
  return e == cudaSuccess ? n : 0;
}
