// Fused stationary GEMM for sm_100a.
//
// One persistent CTA per SM executes a table of tasks
//     C_region (+)= sum_s  A_slice[s] @ B_slice[s]
// that the host lowered from a Stationary-B / Stationary-C plan.  Per CTA:
//
//   warp 0      TMA producer: waits for staged chunks, fills the smem ring (4 or 3 stages)
//               (A 128x64 K-major, B 64x256 N-major, 128-byte swizzle).
//   warp 1      UMMA issuer: tcgen05.mma 128x256x16 bf16 -> fp32 accumulators in
//               TMEM (two 256-column buffers, so the epilogue of tile i overlaps
//               the main loop of tile i+1); owns TMEM allocation.
//   warps 2-9   epilogue: tcgen05.ld -> registers -> shared-memory transpose -> C, two
//               warps per TMEM lane quadrant, each draining half of the tile's columns.
//               C may live in a peer's memory; then the partial tile is stored or
//               pushed with red.global.add (the remote accumulate of Stationary-B
//               and of replica reduction).
//   warps 10-13 fetch warps: copy remote (peer memory, plain P2P loads) or
//               misaligned operand slices into a local staging buffer, piece by
//               piece, and bump a per-chunk counter; the producer of whichever
//               CTA needs the chunk waits on that counter before its TMA loads.
//               TMA therefore only ever reads this GPU's own memory.
//
// Every wait is bounded by UgFusedParams::timeout_ns; a timeout records a code in
// the status word, raises a CTA-wide abort flag and the CTA drains and returns.
//
// Counterpart in the reference: the host loops of stationary_c_plan.py:358-523
// and stationary_b_plan.py:340-564 (get_tile_async + torch.addmm / torch.mm +
// accumulate_tile), and accumulate_kernels.py:12-35 for the remote add.
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

#include "fused_common.cuh"

using namespace ugptx;
using namespace ugfused;

namespace {


// Two tile shapes share the kernel source:
//   BM = 128: tile 128 x 256, 4 stages of 48 KiB, two accumulators (epilogue overlaps the next main loop);
//             96 operand bytes per tensor cycle - best when a tile has few K blocks.
//   BM = 256: tile 256 x 256 as two 128-row UMMAs that share the B stage, 3 stages of 64 KiB, one accumulator
//             pair filling TMEM (the epilogue is exposed); 64 operand bytes per tensor cycle, and a stage feeds
//             1024 tensor cycles, which covers the issuing thread's per-stage work - best for long K.
template <int BM>
struct Cfg {
  static constexpr int kHalves = BM / 128;
  static constexpr int kStages = BM == 128 ? 4 : 3;
  static constexpr int kAccBufs = BM == 128 ? 2 : 1;
  static constexpr uint32_t kABytes = BM * UG_BK * 2;
  static constexpr uint32_t kStageBytes = kABytes + kBBytes;
  static constexpr uint32_t kRingBytes = kStages * kStageBytes;
  static constexpr uint32_t kSmemBytes = kRingBytes + 1024 /*alignment slack*/ + kCtlBytes + kEpiBytes;
};

struct Shared {
  uint64_t full[UG_STAGES];
  uint64_t empty[UG_STAGES];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  volatile uint32_t abort;
  TileQueue tq;
};
static_assert(sizeof(Shared) <= kCtlBytes, "control block overlaps the epilogue buffers");

template <int BM>
__global__ void __launch_bounds__(kNumThreads, 1) ug_fused_gemm_kernel(const UgFusedParams P) {
  using C = Cfg<BM>;
  constexpr uint32_t kABytes = C::kABytes;
  constexpr uint32_t kStageBytes = C::kStageBytes;
  constexpr uint32_t kRingBytes = C::kRingBytes;
  constexpr uint32_t kStages = C::kStages;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t ring = (raw_addr + 1023u) & ~1023u;            // 1024-byte aligned stage ring
  Shared* sh = reinterpret_cast<Shared*>(smem_raw + (ring - raw_addr) + kRingBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const UgTask* __restrict__ tasks = reinterpret_cast<const UgTask*>(P.tasks);
  const UgSegment* __restrict__ segs = reinterpret_cast<const UgSegment*>(P.segs);
  const uint32_t* flags = reinterpret_cast<const uint32_t*>(P.flags);
  const int32_t* __restrict__ flag_need = reinterpret_cast<const int32_t*>(P.flag_need);

  WaitCtl ctl;
  ctl.abort = &sh->abort;
  ctl.status = reinterpret_cast<uint32_t*>(P.status);
  ctl.deadline = global_timer_ns() + P.timeout_ns;
  ctl.peer_abort = 0u;
  // Static schedule: CTA b runs tiles b, b + grid, ...  Dynamic: after its first tile the producer claims the next
  // unclaimed tile from a global counter and hands it to the other roles through sh->tq.
  const bool dyn = P.sched != 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(smem_u32(&sh->full[s]), 1);
      mbar_init(smem_u32(&sh->empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&sh->acc_full[b]), 1);
      mbar_init(smem_u32(&sh->acc_empty[b]), kNumEpiWarps * 32);
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
    tmem_alloc(smem_u32(&sh->tmem_base), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = sh->tmem_base;

  if (warp == kProducerWarp) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      uint64_t seen[4] = {0, 0, 0, 0};   // tensor maps already acquired by this thread
      bool ok = true;
      int tile = blockIdx.x;
      for (int iter = 0; ok; ++iter) {
        if (iter > 0) tile = dyn ? static_cast<int>(gridDim.x + atomicAdd(reinterpret_cast<uint32_t*>(P.sched), 1u))
                                 : tile + static_cast<int>(gridDim.x);
        if (dyn) tileq_publish(&sh->tq, iter, tile);
        if (tile >= P.total_tiles) break;
        const TileCoord tc = locate(tasks, P.num_tasks, tile);
        const UgTask& t = tasks[tc.task];
        if (!task_in_bounds(P, t)) { raise_error(ctl, UG_ERR_BAD_TABLE); break; }
        const int tile_n = task_tile_n(t);
        const int n_rem = min(tile_n, t.n - tc.nt * tile_n);
        const int n_chunks = min(4, (n_rem + 63) >> 6);
        const uint32_t tx_bytes = kABytes + n_chunks * kBChunkBytes;
        trace_put(P, blockIdx.x, iter, UG_TR_TILE, static_cast<uint64_t>(tile) + 1u);
        trace_now(P, blockIdx.x, iter, UG_TR_PROD_BEGIN);
        uint64_t waited = 0;
        for (int s = 0; ok && s < t.seg_count; ++s) {
          const UgSegment& sg = segs[t.seg_begin + s];
          if (!segment_in_bounds(P, sg, sg.a_flag + tc.mt, sg.b_flag + (tc.nt * tile_n) / UG_BN)) {
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
            ok = flag_wait(flags + f, static_cast<uint32_t>(flag_need[f]), ctl);
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
          const int ay = sg.a_row0 + tc.mt * BM;
          const int bx = sg.b_col0 + tc.nt * tile_n;
          for (int kb = 0; kb < nkb; ++kb) {
            ok = mbar_wait(smem_u32(&sh->empty[stage]), phase ^ 1u, ctl);
            if (!ok) break;
            const uint32_t fb = smem_u32(&sh->full[stage]);
            const uint32_t sa = ring + stage * kStageBytes;
            const uint32_t sb = sa + kABytes;
            mbar_arrive_expect_tx(fb, tx_bytes);
            tma_load_2d(sa, amap, sg.a_col0 + kb * UG_BK, ay, fb);
            for (int c = 0; c < n_chunks; ++c)
              tma_load_2d(sb + c * kBChunkBytes, bmap, bx + c * 64, sg.b_row0 + kb * UG_BK, fb);
            if (++stage == kStages) { stage = 0; phase ^= 1u; }
          }
        }
        trace_put(P, blockIdx.x, iter, UG_TR_PROD_FLAGWAIT, waited);
        trace_now(P, blockIdx.x, iter, UG_TR_PROD_END);
      }
    }
  } else if (warp == kMmaWarp) {
    // ------------------------------------------------------------ UMMA issuer
    if (lane == 0) {
      uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
      bool ok = true;
      for (int iter = 0; ok; ++iter) {
        const int tile = dyn ? tileq_get(&sh->tq, iter, ctl) : static_cast<int>(blockIdx.x + iter * gridDim.x);
        if (tile < 0 || tile >= P.total_tiles) break;
        const TileCoord tc = locate(tasks, P.num_tasks, tile);
        const UgTask& t = tasks[tc.task];
        const int n_rem = min(task_tile_n(t), t.n - tc.nt * task_tile_n(t));
        const uint32_t idesc = make_idesc(static_cast<uint32_t>((n_rem + 15) & ~15));
        ok = mbar_wait(smem_u32(&sh->acc_empty[acc]), acc_phase ^ 1u, ctl);
        if (!ok) break;
        tc_fence_after();
        trace_now(P, blockIdx.x, iter, UG_TR_MMA_BEGIN);
        trace_put(P, blockIdx.x, iter, UG_TR_MMA_CLK, static_cast<uint64_t>(clock64()));
        const uint32_t d_tmem = tmem_base + (C::kAccBufs == 2 ? acc * UG_BN : 0u);
        for (int kb = 0; kb < t.kblocks; ++kb) {
          ok = mbar_wait(smem_u32(&sh->full[stage]), phase, ctl);
          if (!ok) break;
          tc_fence_after();
          const uint32_t sa = ring + stage * kStageBytes;
          const uint32_t sb = sa + kABytes;
#pragma unroll
          for (int ks = 0; ks < UG_BK / 16; ++ks) {
            const uint64_t bd = make_desc_b(sb + ks * 2048);
#pragma unroll
            for (int h = 0; h < C::kHalves; ++h) {
              const uint64_t ad = make_desc_a(sa + h * (128 * UG_BK * 2) + ks * 32);
              umma_bf16(d_tmem + h * UG_BN, ad, bd, idesc, (kb > 0 || ks > 0) ? 1u : 0u);
            }
          }
          umma_commit(smem_u32(&sh->empty[stage]));
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        umma_commit(smem_u32(&sh->acc_full[acc]));
        trace_now(P, blockIdx.x, iter, UG_TR_MMA_ISSUED);
        if (C::kAccBufs == 2) acc ^= 1u;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
  } else if (warp < kFetchWarp0) {
    // ------------------------------------------------------------ epilogue
    const int quad = warp & 3;                       // TMEM lane quadrant this warp may read
    const int part = (warp - kEpiWarp0) >> 2;        // 0: left part of the tile's columns, 1: right part
    const bool tracer = warp == kEpiWarp0 && lane == 0;
    float* epi_buf = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(sh) + kCtlBytes) + (warp - kEpiWarp0) * (kEpiWarpBytes / 4);
    uint32_t acc = 0, acc_phase = 0;
    bool ok = true;
    for (int iter = 0; ok; ++iter) {
      const int tile = dyn ? tileq_get(&sh->tq, iter, ctl) : static_cast<int>(blockIdx.x + iter * gridDim.x);
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
      // the two warps of a quadrant split the columns on a multiple of 64 (whole 128-byte row segments each)
      const int split = min(n_rem, ((n_rem + 127) >> 7) << 6);
      const int c0 = part == 0 ? 0 : split, cn = part == 0 ? split : n_rem - split;
      float csum = 0.f;
      float* acc_sum = P.checksum != 0 ? &csum : nullptr;
#pragma unroll
      for (int h = 0; h < C::kHalves; ++h) {
        if (cn <= 0 || tc.mt * BM + h * 128 >= t.m) break;     // nothing to do (warp-uniform)
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) +
                               (C::kAccBufs == 2 ? acc * UG_BN : static_cast<uint32_t>(h) * UG_BN);
        epilogue_drain(taddr + c0, t, tc.mt * BM + h * 128 + quad * 32, col0 + c0, cn, UG_BN - c0, epi_buf, lane, acc_sum);
      }
      if (tracer) trace_now(P, blockIdx.x, iter, UG_TR_EPI_END);
      tc_fence_before();
      mbar_arrive(smem_u32(&sh->acc_empty[acc]));
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
    // Give copies and MMAs already in flight time to land before smem / TMEM go away.
    const uint64_t until = global_timer_ns() + 200000ull;
    while (global_timer_ns() < until) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == kMmaWarp) tmem_dealloc(tmem_base, kTmemCols);
  if (threadIdx.x == 0 && dyn) {
    // Every role of this CTA is done, so it claims no more tiles: the last CTA to get here re-arms the counters.
    uint32_t* sched = reinterpret_cast<uint32_t*>(P.sched);
    if (atomicAdd(sched + 1, 1u) == gridDim.x - 1) {
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

extern "C" int ug_fused_gemm_smem_bytes(void) { return static_cast<int>(Cfg<256>::kSmemBytes); }

namespace {
template <int BM>
int launch_fused(const UgFusedParams* params, int grid, cudaStream_t stream, int dev) {
  static bool configured[64] = {};
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(ug_fused_gemm_kernel<BM>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(Cfg<BM>::kSmemBytes));
    if (e != cudaSuccess) return static_cast<int>(e);
    configured[dev] = true;
  }
  ug_fused_gemm_kernel<BM><<<grid, kNumThreads, Cfg<BM>::kSmemBytes, stream>>>(*params);
  return static_cast<int>(cudaGetLastError());
}
}  // namespace

extern "C" int ug_fused_gemm(const UgFusedParams* params, int grid, void* stream) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (grid <= 0) return static_cast<int>(cudaErrorInvalidValue);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (params->tile_m == 256) return launch_fused<256>(params, grid, st, dev);
  if (params->tile_m == 0 || params->tile_m == 128) return launch_fused<128>(params, grid, st, dev);
  return static_cast<int>(cudaErrorInvalidValue);
}
