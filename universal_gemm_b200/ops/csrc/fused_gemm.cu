// Fused stationary GEMM for sm_100a.
//
// One persistent CTA per SM executes a table of tasks
//     C_region (+)= sum_s  A_slice[s] @ B_slice[s]
// that the host lowered from a Stationary-B / Stationary-C plan.  Per CTA:
//
//   warp 0      TMA producer: waits for staged chunks, fills a 4-deep smem ring
//               (A 128x64 K-major, B 64x256 N-major, 128-byte swizzle).
//   warp 1      UMMA issuer: tcgen05.mma 128x256x16 bf16 -> fp32 accumulators in
//               TMEM (two 256-column buffers, so the epilogue of tile i overlaps
//               the main loop of tile i+1); owns TMEM allocation.
//   warps 2-5   epilogue: tcgen05.ld -> registers -> C.  C may live in a peer's
//               memory; then the partial tile is pushed with red.global.add
//               (the remote accumulate of Stationary-B and of replica reduction).
//   warps 6-9   fetch warps: copy remote (peer memory, plain P2P loads) or
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

#include "ptx_sm100.cuh"
#include "ugemm_b200.h"

using namespace ugptx;

namespace {

constexpr int kNumThreads = 320;
constexpr int kProducerWarp = 0;
constexpr int kMmaWarp = 1;
constexpr int kFetchWarp0 = 6;  // warps 2..5 are the epilogue, 6..9 fetch

constexpr uint32_t kBChunkBytes = UG_BK * 64 * 2;      // 8 KiB: 64 k rows x 64 n elements
constexpr uint32_t kBBytes = 4 * kBChunkBytes;         // 32 KiB
constexpr uint32_t kEpiRowFloats = 36;                 // 32 columns + 4 of padding: conflict-free v4 rows
constexpr uint32_t kEpiWarpBytes = 32 * kEpiRowFloats * 4;
constexpr uint32_t kEpiBytes = 4 * kEpiWarpBytes;      // one transpose buffer per epilogue warp
constexpr uint32_t kTmemCols = 512;                    // 128 lanes x 512 fp32 columns: all of TMEM

// Two tile shapes share the kernel source:
//   BM = 128: tile 128 x 256, 4 stages of 48 KiB, two accumulators (epilogue overlaps the next main loop);
//             96 operand bytes per tensor cycle - best when a tile has few K blocks.
//   BM = 256: tile 256 x 256 as two 128-row UMMAs that share the B stage, 3 stages of 64 KiB, one accumulator
//             pair filling TMEM; 64 operand bytes per tensor cycle and 1.5 x the latency cover - best for long K.
template <int BM>
struct Cfg {
  static constexpr int kHalves = BM / 128;
  static constexpr int kStages = BM == 128 ? 4 : 3;
  static constexpr int kAccBufs = BM == 128 ? 2 : 1;
  static constexpr uint32_t kABytes = BM * UG_BK * 2;
  static constexpr uint32_t kStageBytes = kABytes + kBBytes;
  static constexpr uint32_t kRingBytes = kStages * kStageBytes;
  static constexpr uint32_t kSmemBytes = kRingBytes + 1024 /*alignment slack*/ + 256 /*barriers*/ + kEpiBytes;
};

struct Shared {
  uint64_t full[UG_STAGES];
  uint64_t empty[UG_STAGES];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  volatile uint32_t abort;
};

struct WaitCtl {
  volatile uint32_t* abort;
  uint32_t* status;
  uint64_t deadline;
};

__device__ __forceinline__ void raise_error(const WaitCtl& ctl, uint32_t code) {
  atomicCAS(ctl.status, 0u, code);
  *ctl.abort = 1u;
}

// Bounded mbarrier wait.  Returns false after an abort or a timeout.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, const WaitCtl& ctl) {
  uint32_t spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++spins & 0xffu) == 0u) {
      if (*ctl.abort) return false;
      if (global_timer_ns() > ctl.deadline) {
        raise_error(ctl, UG_ERR_TIMEOUT_MBAR);
        return false;
      }
    }
  }
  return true;
}

// Bounded wait until counter >= need (a staged chunk has fully landed).
__device__ __forceinline__ bool flag_wait(const uint32_t* counter, uint32_t need, const WaitCtl& ctl) {
  uint32_t spins = 0;
  while (ld_acquire_gpu(counter) < need) {
    __nanosleep(64);
    if ((++spins & 0x3fu) == 0u) {
      if (*ctl.abort) return false;
      if (global_timer_ns() > ctl.deadline) {
        raise_error(ctl, UG_ERR_TIMEOUT_FLAG);
        return false;
      }
    }
  }
  return true;
}

struct TileCoord {
  int task;
  int mt, nt;
};

__device__ __forceinline__ int find_task(const UgTask* __restrict__ tasks, int num_tasks, int tile) {
  int lo = 0, hi = num_tasks - 1;
  while (lo < hi) {
    int mid = (lo + hi + 1) >> 1;
    if (tasks[mid].tile_begin <= tile) lo = mid; else hi = mid - 1;
  }
  return lo;
}

// Banded raster: inside a band of group_m tile rows, m runs fastest so the A band
// stays in L2 while the CTAs sweep across n.
__device__ __forceinline__ TileCoord locate(const UgTask* __restrict__ tasks, int num_tasks, int tile) {
  TileCoord tc;
  tc.task = find_task(tasks, num_tasks, tile);
  const UgTask& t = tasks[tc.task];
  int idx = tile - t.tile_begin;
  int gm = t.group_m > 0 ? t.group_m : t.m_tiles;
  int band_tiles = gm * t.n_tiles;
  int band = idx / band_tiles;
  int first_m = band * gm;
  int band_m = min(gm, t.m_tiles - first_m);
  int rem = idx - band * band_tiles;
  tc.mt = first_m + rem % band_m;
  tc.nt = rem / band_m;
  return tc;
}

// UMMA shared-memory descriptors (sm_100 format, version 1, 128-byte swizzle).
// A tile: K-major, rows of 128 bytes, 8-row groups 1024 bytes apart (SBO).
__device__ __forceinline__ uint64_t make_desc_a(uint32_t saddr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr >> 4) & 0x3fffu);
  d |= static_cast<uint64_t>(1u) << 16;                  // LBO (unused for swizzled K-major)
  d |= static_cast<uint64_t>(1024u >> 4) << 32;          // SBO
  d |= static_cast<uint64_t>(1u) << 46;                  // descriptor version
  d |= static_cast<uint64_t>(2u) << 61;                  // SWIZZLE_128B
  return d;
}
// B tile: N-major.  One k row = 64 n elements = 128 bytes; 8-k-row groups are 1024
// bytes apart (SBO); the next 64 n elements start kBChunkBytes later (LBO).
__device__ __forceinline__ uint64_t make_desc_b(uint32_t saddr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr >> 4) & 0x3fffu);
  d |= static_cast<uint64_t>(kBChunkBytes >> 4) << 16;   // LBO
  d |= static_cast<uint64_t>(1024u >> 4) << 32;          // SBO
  d |= static_cast<uint64_t>(1u) << 46;
  d |= static_cast<uint64_t>(2u) << 61;
  return d;
}
// Instruction descriptor: D fp32, A/B bf16, A K-major, B MN-major, M = 128, N = n.
__device__ __forceinline__ uint32_t make_idesc(uint32_t n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (0u << 15) | (1u << 16) | ((n >> 3) << 17) |
         ((static_cast<uint32_t>(UG_BM) >> 4) << 24);
}

// ---------------------------------------------------------------- epilogue stores
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

// Write 32 consecutive accumulator columns of one row.  `ncols` (1..32) of them are
// inside the region.  `p` points at the first of them.
__device__ __forceinline__ void store_row_f32(float* p, const uint32_t (&v)[32], int ncols, int mode,
                                              bool vec) {
  if (vec && ncols == 32) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float a = __uint_as_float(v[4 * j + 0]), b = __uint_as_float(v[4 * j + 1]);
      float c = __uint_as_float(v[4 * j + 2]), d = __uint_as_float(v[4 * j + 3]);
      float4* q = reinterpret_cast<float4*>(p + 4 * j);
      if (mode == 1) {
        red_add_v4_f32(q, a, b, c, d);
      } else {
        if (mode == 0) {
          float4 old = *q;
          a += old.x; b += old.y; c += old.z; d += old.w;
        }
        *q = make_float4(a, b, c, d);
      }
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      if (j < ncols) {
        float a = __uint_as_float(v[j]);
        if (mode == 1) red_add_f32(p + j, a);
        else if (mode == 0) p[j] += a;
        else p[j] = a;
      }
    }
  }
}

__device__ __forceinline__ void store_row_bf16(__nv_bfloat16* p, const uint32_t (&v)[32], int ncols,
                                               int mode, bool vec) {
  if (vec && ncols == 32) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float f[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(v[8 * j + e]);
      uint4* q = reinterpret_cast<uint4*>(p + 8 * j);
      if (mode == 1) {
        red_add_v4_bf16x2(q, pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]),
                          pack_bf16x2(f[6], f[7]));
      } else {
        if (mode == 0) {
          uint4 old = *q;
          const __nv_bfloat162* o = reinterpret_cast<const __nv_bfloat162*>(&old);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            float2 of = __bfloat1622float2(o[e]);
            f[2 * e] += of.x;
            f[2 * e + 1] += of.y;
          }
        }
        uint4 out;
        out.x = pack_bf16x2(f[0], f[1]); out.y = pack_bf16x2(f[2], f[3]);
        out.z = pack_bf16x2(f[4], f[5]); out.w = pack_bf16x2(f[6], f[7]);
        *q = out;
      }
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      if (j < ncols) {
        float a = __uint_as_float(v[j]);
        if (mode == 1) atomicAdd(p + j, __float2bfloat16_rn(a));
        else if (mode == 0) p[j] = __float2bfloat16_rn(__bfloat162float(p[j]) + a);
        else p[j] = __float2bfloat16_rn(a);
      }
    }
  }
}

// Coalesced variant for full, 16-byte aligned chunks: the warp's 32 x 32 block goes through a
// shared-memory buffer so that each store / reduction instruction covers whole 128-byte row
// segments (4 rows of fp32, 8 rows of bf16) instead of 32 different rows.  This matters most for
// red.add into a peer's memory, where every instruction becomes a few full NVLink packets.
__device__ __forceinline__ void store_chunk_f32(float* sb, const uint32_t (&v)[32], int lane, float* c_base,
                                                int64_t ldc, int rows_valid, int mode) {
#pragma unroll
  for (int j = 0; j < 8; ++j)
    *reinterpret_cast<uint4*>(sb + lane * kEpiRowFloats + 4 * j) = make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
  __syncwarp();
  const int rsub = lane >> 3, cseg = (lane & 7) * 4;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int r = i * 4 + rsub;
    if (r < rows_valid) {
      float4 x = *reinterpret_cast<const float4*>(sb + r * kEpiRowFloats + cseg);
      float4* g = reinterpret_cast<float4*>(c_base + r * ldc + cseg);
      if (mode == 1) {
        red_add_v4_f32(g, x.x, x.y, x.z, x.w);
      } else {
        if (mode == 0) {
          const float4 old = *g;
          x.x += old.x; x.y += old.y; x.z += old.z; x.w += old.w;
        }
        *g = x;
      }
    }
  }
  __syncwarp();
}

__device__ __forceinline__ void store_chunk_bf16(float* sbf, const uint32_t (&v)[32], int lane,
                                                 __nv_bfloat16* c_base, int64_t ldc, int rows_valid, int mode) {
  // 64 payload bytes per row, rows 80 bytes apart.
  unsigned char* sb = reinterpret_cast<unsigned char*>(sbf);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    uint4 q;
    q.x = pack_bf16x2(__uint_as_float(v[8 * j + 0]), __uint_as_float(v[8 * j + 1]));
    q.y = pack_bf16x2(__uint_as_float(v[8 * j + 2]), __uint_as_float(v[8 * j + 3]));
    q.z = pack_bf16x2(__uint_as_float(v[8 * j + 4]), __uint_as_float(v[8 * j + 5]));
    q.w = pack_bf16x2(__uint_as_float(v[8 * j + 6]), __uint_as_float(v[8 * j + 7]));
    *reinterpret_cast<uint4*>(sb + lane * 80 + j * 16) = q;
  }
  __syncwarp();
  const int rsub = lane >> 2, cseg = (lane & 3) * 8;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = i * 8 + rsub;
    if (r < rows_valid) {
      uint4 x = *reinterpret_cast<const uint4*>(sb + r * 80 + (lane & 3) * 16);
      uint4* g = reinterpret_cast<uint4*>(c_base + r * ldc + cseg);
      if (mode == 1) {
        red_add_v4_bf16x2(g, x.x, x.y, x.z, x.w);
      } else {
        if (mode == 0) {
          const uint4 old = *g;
          const __nv_bfloat162* o = reinterpret_cast<const __nv_bfloat162*>(&old);
          __nv_bfloat162* n = reinterpret_cast<__nv_bfloat162*>(&x);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 a = __bfloat1622float2(n[e]), b = __bfloat1622float2(o[e]);
            n[e] = __floats2bfloat162_rn(a.x + b.x, a.y + b.y);
          }
        }
        *g = x;
      }
    }
  }
  __syncwarp();
}

// ---------------------------------------------------------------- fetch warps
// Copy one piece with the 32 lanes of a warp.  mode 0: 16-byte vectors, eight in
// flight per lane.  mode 1: the source is only 2-byte aligned; every 16-byte
// destination vector is gathered from eight 2-byte loads.
__device__ __forceinline__ void copy_piece(const UgPiece& pc, int lane) {
  const int vec_per_row = (pc.row_bytes + 15) >> 4;
  const int64_t total = static_cast<int64_t>(pc.rows) * vec_per_row;
  const char* src = reinterpret_cast<const char*>(pc.src);
  char* dst = reinterpret_cast<char*>(pc.dst);
  if (pc.mode == 0) {
    // Lanes run along a row, U rows are in flight per lane.  All loads of a batch are issued before
    // the first store (the compiler barrier keeps the two phases apart), so one warp keeps
    // U x 512 bytes on the wire.
    constexpr int U = 16;
    for (int r0 = 0; r0 < pc.rows; r0 += U) {
      for (int c = lane; c < vec_per_row; c += 32) {
        uint4 buf[U];
        const char* s0 = src + static_cast<int64_t>(r0) * pc.src_ld + (static_cast<int64_t>(c) << 4);
#pragma unroll
        for (int u = 0; u < U; ++u)
          if (r0 + u < pc.rows) buf[u] = ld_stream_v4(s0 + u * pc.src_ld);
        asm volatile("" ::: "memory");
        char* d0 = dst + static_cast<int64_t>(r0) * pc.dst_ld + (static_cast<int64_t>(c) << 4);
#pragma unroll
        for (int u = 0; u < U; ++u)
          if (r0 + u < pc.rows) *reinterpret_cast<uint4*>(d0 + u * pc.dst_ld) = buf[u];
      }
    }
  } else {
    for (int64_t i = lane; i < total; i += 32) {
      int r = static_cast<int>(i / vec_per_row);
      int c = static_cast<int>(i - static_cast<int64_t>(r) * vec_per_row);
      const uint16_t* s = reinterpret_cast<const uint16_t*>(src + r * pc.src_ld + (static_cast<int64_t>(c) << 4));
      int valid = min(8, (pc.row_bytes - (c << 4)) >> 1);
      uint16_t e[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) e[k] = (k < valid) ? s[k] : static_cast<uint16_t>(0);
      uint4 out;
      out.x = e[0] | (static_cast<uint32_t>(e[1]) << 16);
      out.y = e[2] | (static_cast<uint32_t>(e[3]) << 16);
      out.z = e[4] | (static_cast<uint32_t>(e[5]) << 16);
      out.w = e[6] | (static_cast<uint32_t>(e[7]) << 16);
      *reinterpret_cast<uint4*>(dst + r * pc.dst_ld + (static_cast<int64_t>(c) << 4)) = out;
    }
  }
}

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

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(smem_u32(&sh->full[s]), 1);
      mbar_init(smem_u32(&sh->empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&sh->acc_full[b]), 1);
      mbar_init(smem_u32(&sh->acc_empty[b]), 128);
    }
    sh->abort = 0;
    fence_mbar_init();
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
      for (int tile = blockIdx.x; ok && tile < P.total_tiles; tile += gridDim.x) {
        const TileCoord tc = locate(tasks, P.num_tasks, tile);
        const UgTask& t = tasks[tc.task];
        const int n_rem = t.n - tc.nt * UG_BN;
        const int n_chunks = min(4, (n_rem + 63) >> 6);
        const uint32_t tx_bytes = kABytes + n_chunks * kBChunkBytes;
        for (int s = 0; ok && s < t.seg_count; ++s) {
          const UgSegment& sg = segs[t.seg_begin + s];
          if (sg.a_flag >= 0) {
            const int f = sg.a_flag + tc.mt;
            ok = flag_wait(flags + f, static_cast<uint32_t>(flag_need[f]), ctl);
          }
          if (ok && sg.b_flag >= 0) {
            const int f = sg.b_flag + tc.nt;
            ok = flag_wait(flags + f, static_cast<uint32_t>(flag_need[f]), ctl);
          }
          if (!ok) break;
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
          const int bx = sg.b_col0 + tc.nt * UG_BN;
          for (int kb = 0; kb < nkb; ++kb) {
            // Pull the operands of a later K block into L2 now: all CTAs walk K in step, so the first
            // toucher of a line would otherwise pay the DRAM latency inside the smem ring's short cover.
            if (P.prefetch_kblocks > 0 && kb + P.prefetch_kblocks < nkb) {
              const int pk = (kb + P.prefetch_kblocks) * UG_BK;
              tma_prefetch_l2_2d(amap, sg.a_col0 + pk, ay);
              for (int c = 0; c < n_chunks; ++c) tma_prefetch_l2_2d(bmap, bx + c * 64, sg.b_row0 + pk);
            }
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
      }
    }
  } else if (warp == kMmaWarp) {
    // ------------------------------------------------------------ UMMA issuer
    if (lane == 0) {
      uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < P.total_tiles; tile += gridDim.x) {
        const TileCoord tc = locate(tasks, P.num_tasks, tile);
        const UgTask& t = tasks[tc.task];
        const int n_rem = min(UG_BN, t.n - tc.nt * UG_BN);
        const uint32_t idesc = make_idesc(static_cast<uint32_t>((n_rem + 15) & ~15));
        ok = mbar_wait(smem_u32(&sh->acc_empty[acc]), acc_phase ^ 1u, ctl);
        if (!ok) break;
        tc_fence_after();
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
        if (C::kAccBufs == 2) acc ^= 1u;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
  } else if (warp < kFetchWarp0) {
    // ------------------------------------------------------------ epilogue
    const int quad = warp & 3;   // TMEM lane quadrant this warp may read
    float* epi_buf = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(sh) + 256) + quad * (kEpiWarpBytes / 4);
    uint32_t acc = 0, acc_phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < P.total_tiles; tile += gridDim.x) {
      const TileCoord tc = locate(tasks, P.num_tasks, tile);
      const UgTask& t = tasks[tc.task];
      ok = mbar_wait(smem_u32(&sh->acc_full[acc]), acc_phase, ctl);
      if (!ok) break;
      tc_fence_after();
      const int col0 = tc.nt * UG_BN;
      const int n_rem = min(UG_BN, t.n - col0);
#pragma unroll
      for (int h = 0; h < C::kHalves; ++h) {
        const int row = tc.mt * BM + h * 128 + quad * 32 + lane;
        const bool row_ok = row < t.m;
        if (tc.mt * BM + h * 128 >= t.m) break;       // whole half outside the region (warp-uniform)
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) +
                               (C::kAccBufs == 2 ? acc * UG_BN : static_cast<uint32_t>(h) * UG_BN);
        for (int c = 0; c < n_rem; c += 32) {
          uint32_t v[32];
          tmem_ld_32x32(taddr + c, v);
          tmem_ld_wait();
          const int ncols = min(32, n_rem - c);
          const int row0 = tc.mt * BM + h * 128 + quad * 32;          // first row of this warp
          if (t.c_vec != 0 && ncols == 32) {
            const int rows_valid = min(32, t.m - row0);               // <= 0 when the warp is past the region
            const int64_t off0 = static_cast<int64_t>(row0) * t.ldc + col0 + c;
            if (t.c_dtype == 0)
              store_chunk_f32(epi_buf, v, lane, reinterpret_cast<float*>(t.c_ptr) + off0, t.ldc, rows_valid, t.c_mode);
            else
              store_chunk_bf16(epi_buf, v, lane, reinterpret_cast<__nv_bfloat16*>(t.c_ptr) + off0, t.ldc, rows_valid,
                               t.c_mode);
          } else if (row_ok) {
            const int64_t off = static_cast<int64_t>(row) * t.ldc + col0 + c;
            if (t.c_dtype == 0)
              store_row_f32(reinterpret_cast<float*>(t.c_ptr) + off, v, ncols, t.c_mode, false);
            else
              store_row_bf16(reinterpret_cast<__nv_bfloat16*>(t.c_ptr) + off, v, ncols, t.c_mode, false);
          }
        }
      }
      tc_fence_before();
      mbar_arrive(smem_u32(&sh->acc_empty[acc]));
      if (C::kAccBufs == 2) acc ^= 1u;
      if (acc == 0) acc_phase ^= 1u;
    }
  } else {
    // ------------------------------------------------------------ fetch warps
    const UgPiece* __restrict__ pieces = reinterpret_cast<const UgPiece*>(P.pieces);
    uint32_t* counter = reinterpret_cast<uint32_t*>(P.piece_counter);
    uint32_t* wflags = reinterpret_cast<uint32_t*>(P.flags);
    while (P.num_pieces > 0) {
      uint32_t p = 0;
      if (lane == 0) p = atomicAdd(counter, 1u);
      p = __shfl_sync(0xffffffffu, p, 0);
      if (p >= static_cast<uint32_t>(P.num_pieces) || sh->abort) break;
      const UgPiece pc = pieces[p];
      copy_piece(pc, lane);
      __threadfence();
      __syncwarp();
      if (lane == 0) {
        __threadfence();
        red_release_gpu_add(wflags + pc.flag, 1u);
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
