// Device helpers shared by the fused GEMM kernels (one-CTA tiles in fused_gemm.cu, CTA-pair tiles in
// fused_gemm_pair.cu): bounded waits, tile raster, UMMA descriptors, epilogue stores, fetch-warp copy.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

#include "ptx_sm100.cuh"
#include "ugemm_b200.h"

namespace ugfused {

using namespace ugptx;

constexpr int kNumThreads = 448;      // 14 warps: producer, UMMA, 8 epilogue, 4 fetch
constexpr int kProducerWarp = 0;
constexpr int kMmaWarp = 1;
constexpr int kEpiWarp0 = 2;    // warps 2..9 are the epilogue: two per TMEM lane quadrant (warp & 3), the first
constexpr int kNumEpiWarps = 8; // four drain the left part of a tile's columns, the other four the right part
constexpr int kFetchWarp0 = 10; // warps 10..13 fetch

constexpr uint32_t kBChunkBytes = UG_BK * 64 * 2;      // 8 KiB: 64 k rows x 64 n elements
constexpr uint32_t kBBytes = 4 * kBChunkBytes;         // 32 KiB
constexpr uint32_t kEpiWarpBytes = 32 * 128;           // 32 rows of 128 bytes, 16-byte groups XOR-swizzled by row
constexpr uint32_t kEpiBytes = kNumEpiWarps * kEpiWarpBytes;   // one transpose buffer per epilogue warp
constexpr uint32_t kCtlBytes = 512;                    // barriers, flags and the tile queue; the epilogue buffers follow
constexpr uint32_t kTmemCols = 512;                    // 128 lanes x 512 fp32 columns: all of TMEM

struct WaitCtl {
  volatile uint32_t* abort;
  uint32_t* status;
  uint64_t deadline;
  uint32_t peer_abort;   // shared::cluster address of the abort word of the other CTA of a pair (0: no partner)
};

// First error wins the status word; the CTA (and its partner in a CTA pair, which would otherwise only leave when
// its own waits run out) drains and returns.  The partner cannot have exited yet: both CTAs meet at a cluster
// barrier before they leave.
__device__ __forceinline__ void raise_error(const WaitCtl& ctl, uint32_t code) {
  atomicCAS(ctl.status, 0u, code);
  *ctl.abort = 1u;
  if (ctl.peer_abort != 0u) st_shared_cluster_u32(ctl.peer_abort, 1u);
}

// In-kernel check of the work tables (UG_ERR_BAD_TABLE): indices a tile is about to use must lie inside the tables
// the launch declared.  A failed check records the error and the tile is never touched.
__device__ __forceinline__ bool task_in_bounds(const UgFusedParams& P, const UgTask& t) {
  return t.seg_begin >= 0 && t.seg_count >= 0 && t.seg_begin + t.seg_count <= P.num_segs;
}
__device__ __forceinline__ bool segment_in_bounds(const UgFusedParams& P, const UgSegment& sg, int a_flag_last,
                                                  int b_flag_last) {
  return sg.a_map >= 0 && sg.a_map < P.num_maps && sg.b_map >= 0 && sg.b_map < P.num_maps && sg.k_len > 0 &&
         (sg.a_flag < 0 || a_flag_last < P.num_flags) && (sg.b_flag < 0 || b_flag_last < P.num_flags);
}

// Optional timeline (UgFusedParams::trace != 0): one 64-byte record per (CTA, tile iteration), written by
// single threads with plain stores; the host reads it after the kernel.  Costs one uniform branch when off.
__device__ __forceinline__ uint64_t* trace_slot(const UgFusedParams& P, int cta, int iter) {
  if (P.trace == 0 || iter > P.trace_slots) return nullptr;
  return reinterpret_cast<uint64_t*>(P.trace) + (static_cast<int64_t>(cta) * (P.trace_slots + 1) + iter) * UG_TR_FIELDS;
}
__device__ __forceinline__ void trace_put(const UgFusedParams& P, int cta, int iter, int field, uint64_t v) {
  if (P.trace == 0 || iter >= P.trace_slots) return;
  trace_slot(P, cta, iter)[field] = v;
}
__device__ __forceinline__ void trace_now(const UgFusedParams& P, int cta, int iter, int field) {
  if (P.trace == 0 || iter >= P.trace_slots) return;
  trace_slot(P, cta, iter)[field] = global_timer_ns();
}
// Summary record of the CTA (index trace_slots).
__device__ __forceinline__ uint64_t* trace_summary(const UgFusedParams& P, int cta) {
  return P.trace == 0 ? nullptr : trace_slot(P, cta, P.trace_slots);
}

// Tile hand-off inside a CTA when tiles are claimed dynamically (UgFusedParams::sched): the TMA producer claims the
// tile of iteration i and publishes (i + 1) << 32 | tile in slot i % 16 with one 64-bit store; the UMMA issuer and
// the epilogue warps read it from there.  No role is ever 16 tiles ahead of another (the operand ring and the two
// accumulator buffers bound the lead), so a slot is not overwritten before everyone has read it.
constexpr int kTileQueueSlots = 16;
struct TileQueue {
  volatile unsigned long long slot[kTileQueueSlots];
};
__device__ __forceinline__ unsigned long long tileq_word(int iter, int tile) {
  return (static_cast<unsigned long long>(iter + 1) << 32) | static_cast<uint32_t>(tile);
}
__device__ __forceinline__ void tileq_publish(TileQueue* q, int iter, int tile) {
  q->slot[iter & (kTileQueueSlots - 1)] = tileq_word(iter, tile);
}
// Bounded wait for the tile of iteration `iter`; -1 after an abort or a timeout.
__device__ __forceinline__ int tileq_get(const TileQueue* q, int iter, const WaitCtl& ctl);

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

// The same wait with a pause between polls, for roles that wait a whole main loop (the epilogue warps): fewer
// issue slots and less power spent on polling, at the price of up to `sleep_ns` of wake-up latency.
__device__ __forceinline__ bool mbar_wait_backoff(uint32_t bar, uint32_t parity, const WaitCtl& ctl, uint32_t sleep_ns) {
  uint32_t spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    if (sleep_ns != 0u) __nanosleep(sleep_ns);
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

__device__ __forceinline__ int tileq_get(const TileQueue* q, int iter, const WaitCtl& ctl) {
  const unsigned long long want = static_cast<unsigned long long>(iter + 1);
  uint32_t spins = 0;
  for (;;) {
    const unsigned long long w = q->slot[iter & (kTileQueueSlots - 1)];
    if ((w >> 32) == want) return static_cast<int>(static_cast<uint32_t>(w));
    if ((++spins & 0x3fu) == 0u) {
      if (*ctl.abort) return -1;
      if (global_timer_ns() > ctl.deadline) {
        raise_error(ctl, UG_ERR_TIMEOUT_MBAR);
        return -1;
      }
      __nanosleep(32);
    }
  }
}

// Columns per output tile of a task: UG_BN, or a narrower width stored in the upper half of c_vec
// (used for the last, partly filled wave of tiles); bit 0 of c_vec says whether 16-byte accesses to C are legal.
__device__ __forceinline__ int task_tile_n(const UgTask& t) {
  const int v = t.c_vec >> 16;
  return v > 0 ? v : UG_BN;
}
__device__ __forceinline__ bool task_c_vec(const UgTask& t) { return (t.c_vec & 1) != 0; }
// Bit 1 of c_vec: the row pitch of C is a multiple of 16 bytes (and C is element-aligned), so every row of a region
// has the same alignment phase even when the region starts on an odd column.
__device__ __forceinline__ bool task_c_pitch_vec(const UgTask& t) { return (t.c_vec & 2) != 0; }
// Bit 2 of c_vec: the task's output rows live in several places (a task merged from tasks of different C tiles);
// c_ptr is then the address of a table uint64[m] with the address of every row's first column, and ldc is unused.
// All rows share one 16-byte alignment phase (checked when the table is built).
__device__ __forceinline__ bool task_c_rows_indirect(const UgTask& t) { return (t.c_vec & 4) != 0; }

// Where the 32 rows of an epilogue warp go: rows of one region (base + r * ldc) or rows named by a table.
struct CRows {
  const uint64_t* tab;   // entry of the warp's first row, or nullptr
  float* base;           // first row of the warp at the region's first column (direct), unused with a table
  int64_t ldc;
  int col;               // column offset added to a table entry
  __device__ __forceinline__ float* row(int r) const {
    return tab != nullptr ? reinterpret_cast<float*>(tab[r]) + col : base + r * ldc;
  }
};

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

// Word offset of 16-byte group `group` (0..7) of row `row` in a transpose buffer.  Rows are 128 bytes without
// padding; XOR-ing the group with the row number keeps both phases free of bank conflicts: lanes of a quarter warp
// write the same group of 8 different rows, and read 8 different groups of one row.
__device__ __forceinline__ int epi_off(int row, int group) { return row * 32 + ((group ^ (row & 7)) << 2); }

// Full, 16-byte aligned chunks: the warp's 32 x 32 block of accumulators goes through a
// shared-memory buffer so that each store / reduction instruction covers whole 128-byte row
// segments (4 rows of fp32, 8 rows of bf16) instead of 32 different rows.  This matters most for
// red.add into a peer's memory, where every instruction becomes a few full NVLink packets.
__device__ __forceinline__ void store_chunk_f32(float* sb, const uint32_t (&v)[32], int lane, float* c_base,
                                                int64_t ldc, int rows_valid, int mode) {
#pragma unroll
  for (int j = 0; j < 8; ++j)
    *reinterpret_cast<uint4*>(sb + epi_off(lane, j)) = make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
  __syncwarp();
  const int rsub = lane >> 3, cseg = (lane & 7) * 4;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int r = i * 4 + rsub;
    if (r < rows_valid) {
      float4 x = *reinterpret_cast<const float4*>(sb + epi_off(r, lane & 7));
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

// 64 bf16 columns at a time: rows of 128 payload bytes, so that every store / reduction instruction covers
// four full 128-byte row segments (half-line segments made the NVLink pushes of bf16 partial tiles inefficient).
__device__ __forceinline__ void store_chunk_bf16_64(float* sbf, const uint32_t (&v0)[32], const uint32_t (&v1)[32],
                                                    int lane, __nv_bfloat16* c_base, int64_t ldc, int rows_valid,
                                                    int mode) {
  // rows of 128 payload bytes, swizzled like the fp32 rows
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    uint4 q;
    q.x = pack_bf16x2(__uint_as_float(v0[8 * j + 0]), __uint_as_float(v0[8 * j + 1]));
    q.y = pack_bf16x2(__uint_as_float(v0[8 * j + 2]), __uint_as_float(v0[8 * j + 3]));
    q.z = pack_bf16x2(__uint_as_float(v0[8 * j + 4]), __uint_as_float(v0[8 * j + 5]));
    q.w = pack_bf16x2(__uint_as_float(v0[8 * j + 6]), __uint_as_float(v0[8 * j + 7]));
    *reinterpret_cast<uint4*>(sbf + epi_off(lane, j)) = q;
    q.x = pack_bf16x2(__uint_as_float(v1[8 * j + 0]), __uint_as_float(v1[8 * j + 1]));
    q.y = pack_bf16x2(__uint_as_float(v1[8 * j + 2]), __uint_as_float(v1[8 * j + 3]));
    q.z = pack_bf16x2(__uint_as_float(v1[8 * j + 4]), __uint_as_float(v1[8 * j + 5]));
    q.w = pack_bf16x2(__uint_as_float(v1[8 * j + 6]), __uint_as_float(v1[8 * j + 7]));
    *reinterpret_cast<uint4*>(sbf + epi_off(lane, j + 4)) = q;
  }
  __syncwarp();
  const int rsub = lane >> 3, seg = lane & 7;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int r = i * 4 + rsub;
    if (r < rows_valid) {
      uint4 x = *reinterpret_cast<const uint4*>(sbf + epi_off(r, seg));
      uint4* g = reinterpret_cast<uint4*>(c_base + r * ldc + seg * 8);
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

// Any alignment, any width: the 32 x 32 block goes through shared memory and every instruction handles 32
// consecutive columns of ONE row (a coalesced, possibly misaligned 128-byte / 64-byte segment).  Used when C
// rows are not 16-byte aligned (odd column offsets of odd-shaped partitions) and for ragged right edges.
__device__ __forceinline__ void store_chunk_scalar(float* sb, const uint32_t (&v)[32], int lane, uint64_t c_ptr,
                                                   int64_t elem_off, int64_t ldc, int rows_valid, int ncols, int mode,
                                                   int dtype) {
#pragma unroll
  for (int j = 0; j < 8; ++j)
    *reinterpret_cast<uint4*>(sb + epi_off(lane, j)) = make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
  __syncwarp();
  if (lane < ncols) {
    for (int r = 0; r < rows_valid; ++r) {
      const float x = sb[epi_off(r, lane >> 2) + (lane & 3)];
      const int64_t off = elem_off + r * ldc + lane;
      if (dtype == 0) {
        float* g = reinterpret_cast<float*>(c_ptr) + off;
        if (mode == 1) red_add_f32(g, x);
        else if (mode == 0) *g += x;
        else *g = x;
      } else {
        __nv_bfloat16* g = reinterpret_cast<__nv_bfloat16*>(c_ptr) + off;
        if (mode == 1) atomicAdd(g, __float2bfloat16_rn(x));
        else if (mode == 0) *g = __float2bfloat16_rn(__bfloat162float(*g) + x);
        else *g = __float2bfloat16_rn(x);
      }
    }
  }
  __syncwarp();
}

// Sum of the accumulator columns [lo, hi) of this lane's row (the checksum a launch can ask for).
__device__ __forceinline__ float sum_columns(const uint32_t (&v)[32], int lo, int hi) {
  float s = 0.f;
#pragma unroll
  for (int j = 0; j < 32; ++j)
    if (j >= lo && j < hi) s += __uint_as_float(v[j]);
  return s;
}

// The same transpose for a 32-column chunk of which only columns [lo, hi) are to be written (lo a multiple of 4;
// c_base 16-byte aligned): whole 16-byte groups inside the range go out as vectors, the ragged end element by element.
__device__ __forceinline__ void store_chunk_f32_ragged(float* sb, const uint32_t (&v)[32], int lane, const CRows& rows,
                                                       int col, int rows_valid, int mode, int lo, int hi) {
#pragma unroll
  for (int j = 0; j < 8; ++j)
    *reinterpret_cast<uint4*>(sb + epi_off(lane, j)) = make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
  __syncwarp();
  const int rsub = lane >> 3, cseg = (lane & 7) * 4;
  if (cseg >= lo && cseg < hi) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int r = i * 4 + rsub;
      if (r < rows_valid) {
        float4 x = *reinterpret_cast<const float4*>(sb + epi_off(r, lane & 7));
        float* g = rows.row(r) + col + cseg;
        if (cseg + 4 <= hi) {
          float4* g4 = reinterpret_cast<float4*>(g);
          if (mode == 1) {
            red_add_v4_f32(g4, x.x, x.y, x.z, x.w);
          } else {
            if (mode == 0) {
              const float4 old = *g4;
              x.x += old.x; x.y += old.y; x.z += old.z; x.w += old.w;
            }
            *g4 = x;
          }
        } else {
          const float xs[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
          for (int e = 0; e < 3; ++e) {
            if (cseg + e < hi) {
              if (mode == 1) red_add_f32(g + e, xs[e]);
              else if (mode == 0) g[e] += xs[e];
              else g[e] = xs[e];
            }
          }
        }
      }
    }
  }
  __syncwarp();
}

// fp32 C whose rows are 16 bytes apart in phase but whose region starts on any column (odd-shaped partitions) and has
// any width: up to three head columns go out element by element, then 32-column chunks that start on a 16-byte
// boundary of C.  `avail` TMEM columns can be read from `taddr`; a last chunk that would read past them is moved back
// by a multiple of four columns and writes only what the chunks before it have not written.
__device__ __forceinline__ void epilogue_drain_f32_shifted(uint32_t taddr, const UgTask& t, int row0, int col0,
                                                           int n_rem, int avail, float* epi_buf, int lane, float* acc) {
  const int rows_valid = min(32, t.m - row0);
  if (rows_valid <= 0) return;
  CRows rows;
  if (task_c_rows_indirect(t)) {
    rows.tab = reinterpret_cast<const uint64_t*>(t.c_ptr) + row0;
    rows.base = nullptr;
    rows.ldc = 0;
    rows.col = col0;
  } else {
    rows.tab = nullptr;
    rows.base = reinterpret_cast<float*>(t.c_ptr) + static_cast<int64_t>(row0) * t.ldc + col0;
    rows.ldc = t.ldc;
    rows.col = 0;
  }
  const int phase = static_cast<int>((reinterpret_cast<uint64_t>(rows.row(0)) >> 2) & 3u);
  const int head = min((4 - phase) & 3, n_rem);
  uint32_t v[32];
  if (head > 0) {
    tmem_ld_32x32(taddr, v);
    tmem_ld_wait();
    if (acc != nullptr && lane < rows_valid) *acc += sum_columns(v, 0, head);
    if (lane < rows_valid) {
      float* g = rows.row(lane);
#pragma unroll
      for (int j = 0; j < 3; ++j) {
        if (j < head) {
          const float x = __uint_as_float(v[j]);
          if (t.c_mode == 1) red_add_f32(g + j, x);
          else if (t.c_mode == 0) g[j] += x;
          else g[j] = x;
        }
      }
    }
  }
  int c = head;
  for (; c < n_rem && c + 32 <= avail; c += 32) {
    tmem_ld_32x32(taddr + c, v);
    tmem_ld_wait();
    if (acc != nullptr && lane < rows_valid) *acc += sum_columns(v, 0, min(32, n_rem - c));
    store_chunk_f32_ragged(epi_buf, v, lane, rows, c, rows_valid, t.c_mode, 0, min(32, n_rem - c));
  }
  if (c < n_rem) {
    // Fewer than 32 columns are left and a chunk on this boundary would read past the readable TMEM columns: move it
    // back by a multiple of four columns (it then skips what is written already); up to three columns can remain
    // beyond its end, they go out element by element from a chunk that ends with the region.
    const int lo = (c + 32 - avail + 3) & ~3;
    const int start = c - lo;
    const int hi = min(32, n_rem - start);
    if (lo < hi) {
      tmem_ld_32x32(taddr + start, v);
      tmem_ld_wait();
      if (acc != nullptr && lane < rows_valid) *acc += sum_columns(v, lo, hi);
      store_chunk_f32_ragged(epi_buf, v, lane, rows, start, rows_valid, t.c_mode, lo, hi);
    }
    const int rem = n_rem - min(start + 32, n_rem);
    if (rem > 0) {
      tmem_ld_32x32(taddr + n_rem - 32, v);
      tmem_ld_wait();
      if (acc != nullptr && lane < rows_valid) *acc += sum_columns(v, 32 - rem, 32);
      if (lane < rows_valid) {
        float* g = rows.row(lane) + n_rem - 32;
#pragma unroll
        for (int j = 29; j < 32; ++j) {
          if (j >= 32 - rem) {
            const float x = __uint_as_float(v[j]);
            if (t.c_mode == 1) red_add_f32(g + j, x);
            else if (t.c_mode == 0) g[j] += x;
            else g[j] = x;
          }
        }
      }
    }
  }
}

// ---------------------------------------------------------------- fetch warps
__device__ __forceinline__ float4 ld_stream_f4(const void* p) {
  const uint4 u = ld_stream_v4(p);
  return make_float4(__uint_as_float(u.x), __uint_as_float(u.y), __uint_as_float(u.z), __uint_as_float(u.w));
}
__device__ __forceinline__ uint16_t ld_stream_u16(const void* p) {
  uint16_t v;
  asm volatile("ld.global.L1::no_allocate.u16 %0, [%1];" : "=h"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ float ld_stream_f1(const void* p) {
  float v;
  asm volatile("ld.global.L1::no_allocate.f32 %0, [%1];" : "=f"(v) : "l"(p));
  return v;
}
// High and low bf16 parts of two fp32 values: hi = bf16(x), lo = bf16(x - hi), packed as bf16x2.
__device__ __forceinline__ void split_bf16x2(float x0, float x1, uint32_t& hi, uint32_t& lo) {
  const __nv_bfloat16 h0 = __float2bfloat16_rn(x0), h1 = __float2bfloat16_rn(x1);
  const __nv_bfloat162 hp = __halves2bfloat162(h0, h1);
  const __nv_bfloat162 lp = __floats2bfloat162_rn(x0 - __bfloat162float(h0), x1 - __bfloat162float(h1));
  hi = *reinterpret_cast<const uint32_t*>(&hp);
  lo = *reinterpret_cast<const uint32_t*>(&lp);
}

// Copy an fp32 piece (possibly from a peer) into two bf16 buffers: the high parts at pc.dst, the low parts
// (pc.mode >> 8) KiB further on.  A 16-byte destination vector holds eight elements, i.e. 32 source bytes.
// `aligned`: source rows start on 16-byte boundaries (two vector loads per destination vector), else 4-byte loads.
// Elements past the end of a row are written as zeros.
__device__ __forceinline__ void copy_piece_split_f32(const UgPiece& pc, int lane, int vec_per_row, uint32_t nvec,
                                                     bool aligned) {
  const char* src = reinterpret_cast<const char*>(pc.src);
  char* dst = reinterpret_cast<char*>(pc.dst);
  const int64_t low = static_cast<int64_t>(static_cast<uint32_t>(pc.mode) >> 8) << 10;
  const uint32_t vpr = static_cast<uint32_t>(vec_per_row);
  const int row_elems = pc.row_bytes >> 1;
  constexpr uint32_t U = 4;                       // destination vectors per lane and batch: 8 x 16 B loads in flight
  for (uint32_t base = 0; base < nvec; base += 32u * U) {
    float f[U][8];
#pragma unroll
    for (uint32_t u = 0; u < U; ++u) {
      const uint32_t idx = min(base + u * 32u + static_cast<uint32_t>(lane), nvec - 1u);
      const uint32_t r = idx / vpr, c = idx - r * vpr;
      const char* sp = src + static_cast<int64_t>(r) * pc.src_ld + (static_cast<int64_t>(c) << 5);
      const int valid = row_elems - static_cast<int>(c << 3);          // elements of this vector inside the row
      if (aligned) {
        const float4 a = ld_stream_f4(sp);
        const float4 b = valid > 4 ? ld_stream_f4(sp + 16) : make_float4(0.f, 0.f, 0.f, 0.f);
        f[u][0] = a.x; f[u][1] = a.y; f[u][2] = a.z; f[u][3] = a.w;
        f[u][4] = b.x; f[u][5] = b.y; f[u][6] = b.z; f[u][7] = b.w;
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) f[u][e] = e < valid ? ld_stream_f1(sp + 4 * e) : 0.f;
      }
#pragma unroll
      for (int e = 0; e < 8; ++e)
        if (e >= valid) f[u][e] = 0.f;
    }
    asm volatile("" ::: "memory");
#pragma unroll
    for (uint32_t u = 0; u < U; ++u) {
      const uint32_t idx = base + u * 32u + static_cast<uint32_t>(lane);
      if (idx < nvec) {
        const uint32_t r = idx / vpr, c = idx - r * vpr;
        uint4 hi, lo;
        split_bf16x2(f[u][0], f[u][1], hi.x, lo.x);
        split_bf16x2(f[u][2], f[u][3], hi.y, lo.y);
        split_bf16x2(f[u][4], f[u][5], hi.z, lo.z);
        split_bf16x2(f[u][6], f[u][7], hi.w, lo.w);
        char* dp = dst + static_cast<int64_t>(r) * pc.dst_ld + (static_cast<int64_t>(c) << 4);
        *reinterpret_cast<uint4*>(dp) = hi;
        *reinterpret_cast<uint4*>(dp + low) = lo;
      }
    }
  }
}

// Mode 0 (16-byte aligned source): the piece is walked as one flat sequence of 16-byte vectors (row after row); a
// warp takes 32 x U consecutive vectors per batch, whatever the piece's shape (one 24 KiB row or 128 rows of 256
// bytes).  The batch is straight-line code: U unconditional loads (lanes past the end re-read the last vector), a
// compiler barrier, then the predicated stores, so one warp keeps U x 512 bytes on the wire: over NVLink the copy
// rate is (bytes in flight) / (about 2 us of latency), and a copy loop whose loads are issued one at a time reaches
// a quarter of the link rate.  U is chosen per launch (UgFusedParams::fetch_depth): loads in flight share the SM's
// outstanding-request capacity with the TMA operand loads, so a plan that needs its remote data slowly asks for less.
template <uint32_t U>
__device__ __forceinline__ void copy_flat_vec(const UgPiece& pc, int lane, int vec_per_row, uint32_t nvec) {
  const char* src = reinterpret_cast<const char*>(pc.src);
  char* dst = reinterpret_cast<char*>(pc.dst);
  const uint32_t vpr = static_cast<uint32_t>(vec_per_row);
  for (uint32_t base = 0; base < nvec; base += 32u * U) {
    uint4 buf[U];
#pragma unroll
    for (uint32_t u = 0; u < U; ++u) {
      const uint32_t idx = min(base + u * 32u + static_cast<uint32_t>(lane), nvec - 1u);
      const uint32_t r = idx / vpr, c = idx - r * vpr;
      buf[u] = ld_stream_v4(src + static_cast<int64_t>(r) * pc.src_ld + (static_cast<int64_t>(c) << 4));
    }
    asm volatile("" ::: "memory");
#pragma unroll
    for (uint32_t u = 0; u < U; ++u) {
      const uint32_t idx = base + u * 32u + static_cast<uint32_t>(lane);
      if (idx < nvec) {
        const uint32_t r = idx / vpr, c = idx - r * vpr;
        *reinterpret_cast<uint4*>(dst + static_cast<int64_t>(r) * pc.dst_ld + (static_cast<int64_t>(c) << 4)) = buf[u];
      }
    }
  }
}

// Copy one piece with the 32 lanes of a warp.  mode 0: 16-byte vectors, sixteen in
// flight per lane.  mode 1: the source is only 2-byte aligned; every 16-byte
// destination vector is gathered from eight 2-byte loads.
__device__ __forceinline__ void copy_piece(const UgPiece& pc, int lane, int depth) {
  const int vec_per_row = (pc.row_bytes + 15) >> 4;
  if (vec_per_row <= 0) return;
  const int64_t total = static_cast<int64_t>(pc.rows) * vec_per_row;
  const char* src = reinterpret_cast<const char*>(pc.src);
  char* dst = reinterpret_cast<char*>(pc.dst);
  const int mode = pc.mode & 0xff;
  if (mode >= 2) {
    copy_piece_split_f32(pc, lane, vec_per_row, static_cast<uint32_t>(total), mode == 2);
    return;
  }
  if (mode == 0) {
    if (depth <= 4) copy_flat_vec<4>(pc, lane, vec_per_row, static_cast<uint32_t>(total));
    else if (depth <= 8) copy_flat_vec<8>(pc, lane, vec_per_row, static_cast<uint32_t>(total));
    else copy_flat_vec<16>(pc, lane, vec_per_row, static_cast<uint32_t>(total));
  } else {
    // Source only 2-byte aligned (odd column offsets or pitches of odd-shaped partitions).  Every 16-byte destination
    // vector is cut out of the two 16-byte-aligned source vectors that cover it (funnel shifts by the source's byte
    // offset), so the copy still moves whole 16-byte vectors over the link: 2-byte loads from a peer cost a 32-byte
    // sector each.  The second vector is only read when it holds needed bytes, so no read leaves the source row.
    // Four destination vectors per lane and batch keep up to eight loads in flight.
    constexpr uint32_t U = 4;
    const uint32_t vpr = static_cast<uint32_t>(vec_per_row);
    const uint32_t nvec = static_cast<uint32_t>(total);
    for (uint32_t base = 0; base < nvec; base += 32u * U) {
      uint4 lo[U], hi[U];
      uint32_t shift[U];
#pragma unroll
      for (uint32_t u = 0; u < U; ++u) {
        const uint32_t idx = min(base + u * 32u + static_cast<uint32_t>(lane), nvec - 1u);
        const uint32_t r = idx / vpr, c = idx - r * vpr;
        const uint64_t sp = reinterpret_cast<uint64_t>(src) + static_cast<uint64_t>(r) * pc.src_ld + (static_cast<uint64_t>(c) << 4);
        const int valid_bytes = min(16, pc.row_bytes - static_cast<int>(c << 4));
        shift[u] = static_cast<uint32_t>(sp & 15u);
        const char* ap = reinterpret_cast<const char*>(sp - shift[u]);
        lo[u] = ld_stream_v4(ap);
        hi[u] = (static_cast<int>(shift[u]) + valid_bytes > 16) ? ld_stream_v4(ap + 16) : make_uint4(0u, 0u, 0u, 0u);
      }
      asm volatile("" ::: "memory");
#pragma unroll
      for (uint32_t u = 0; u < U; ++u) {
        const uint32_t idx = base + u * 32u + static_cast<uint32_t>(lane);
        if (idx < nvec) {
          const uint32_t r = idx / vpr, c = idx - r * vpr;
          const uint32_t w[9] = {lo[u].x, lo[u].y, lo[u].z, lo[u].w, hi[u].x, hi[u].y, hi[u].z, hi[u].w, 0u};
          const uint32_t q = shift[u] >> 2, bits = (shift[u] & 3u) * 8u;
          uint32_t o[4];
#pragma unroll
          for (uint32_t i = 0; i < 4; ++i) {
            uint32_t a = 0u, b = 0u;
#pragma unroll
            for (uint32_t qq = 0; qq < 4; ++qq)
              if (q == qq) { a = w[i + qq]; b = w[i + qq + 1]; }
            o[i] = __funnelshift_r(a, b, bits);
          }
          const int valid = min(8, (pc.row_bytes - static_cast<int>(c << 4)) >> 1);     // elements inside the row
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            if (2 * i >= valid) o[i] = 0u;
            else if (2 * i + 1 >= valid) o[i] &= 0xffffu;
          }
          *reinterpret_cast<uint4*>(dst + static_cast<int64_t>(r) * pc.dst_ld + (static_cast<int64_t>(c) << 4)) =
              make_uint4(o[0], o[1], o[2], o[3]);
        }
      }
    }
  }
}


// Drain this warp's 32 TMEM lanes x n_rem accumulator columns (first column at `taddr`) into rows row0.. and
// columns col0.. of the task's C.  The common case (fp32 C, 16-byte aligned, whole 32-column chunks) is software
// pipelined: the TMEM load of the next chunk is in flight while the current chunk goes through shared memory.
__device__ __forceinline__ void epilogue_drain(uint32_t taddr, const UgTask& t, int row0, int col0, int n_rem,
                                               int avail, float* epi_buf, int lane, float* acc) {
  const int rows_valid = min(32, t.m - row0);               // <= 0 when the warp is past the region
  if (t.c_dtype == 0 && task_c_pitch_vec(t) &&
      (task_c_rows_indirect(t) || !(task_c_vec(t) && (n_rem & 31) == 0 && (col0 & 3) == 0))) {
    epilogue_drain_f32_shifted(taddr, t, row0, col0, n_rem, avail, epi_buf, lane, acc);
    return;
  }
  if (task_c_vec(t) && t.c_dtype == 0 && (n_rem & 31) == 0) {
    float* c_row = reinterpret_cast<float*>(t.c_ptr) + static_cast<int64_t>(row0) * t.ldc + col0;
    uint32_t va[32], vb[32];
    tmem_ld_32x32(taddr, va);
    for (int c = 0; c < n_rem; c += 64) {
      tmem_ld_wait();
      const bool second = c + 32 < n_rem;
      if (second) tmem_ld_32x32(taddr + c + 32, vb);
      if (acc != nullptr && lane < rows_valid) *acc += sum_columns(va, 0, 32);
      store_chunk_f32(epi_buf, va, lane, c_row + c, t.ldc, rows_valid, t.c_mode);
      if (second) {
        tmem_ld_wait();
        if (acc != nullptr && lane < rows_valid) *acc += sum_columns(vb, 0, 32);
        if (c + 64 < n_rem) tmem_ld_32x32(taddr + c + 64, va);
        store_chunk_f32(epi_buf, vb, lane, c_row + c + 32, t.ldc, rows_valid, t.c_mode);
      }
    }
    return;
  }
  for (int c = 0; c < n_rem; c += 32) {
    if (t.c_dtype == 1 && task_c_vec(t) && n_rem - c >= 64) {
      // bf16 output: two 32-column loads make one 128-byte row segment per row
      uint32_t v0[32], v1[32];
      tmem_ld_32x32(taddr + c, v0);
      tmem_ld_32x32(taddr + c + 32, v1);
      tmem_ld_wait();
      if (acc != nullptr && lane < rows_valid) *acc += sum_columns(v0, 0, 32) + sum_columns(v1, 0, 32);
      store_chunk_bf16_64(epi_buf, v0, v1, lane,
                          reinterpret_cast<__nv_bfloat16*>(t.c_ptr) + static_cast<int64_t>(row0) * t.ldc + col0 + c,
                          t.ldc, rows_valid, t.c_mode);
      c += 32;
      continue;
    }
    uint32_t v[32];
    tmem_ld_32x32(taddr + c, v);
    tmem_ld_wait();
    const int ncols = min(32, n_rem - c);
    if (acc != nullptr && lane < rows_valid) *acc += sum_columns(v, 0, ncols);
    const int64_t off0 = static_cast<int64_t>(row0) * t.ldc + col0 + c;
    if (task_c_vec(t) && ncols == 32) {
      if (t.c_dtype == 0)
        store_chunk_f32(epi_buf, v, lane, reinterpret_cast<float*>(t.c_ptr) + off0, t.ldc, rows_valid, t.c_mode);
      else
        store_chunk_bf16(epi_buf, v, lane, reinterpret_cast<__nv_bfloat16*>(t.c_ptr) + off0, t.ldc, rows_valid,
                         t.c_mode);
    } else {
      store_chunk_scalar(epi_buf, v, lane, t.c_ptr, off0, t.ldc, rows_valid, ncols, t.c_mode, t.c_dtype);
    }
  }
}

// Add an epilogue warp's checksum share of one tile to the launch's checksum (a double in device memory).
__device__ __forceinline__ void checksum_flush(uint64_t checksum_ptr, float acc, int lane) {
  if (checksum_ptr == 0) return;
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, d);
  if (lane == 0) atomicAdd(reinterpret_cast<double*>(checksum_ptr), static_cast<double>(acc));
}

}  // namespace ugfused
