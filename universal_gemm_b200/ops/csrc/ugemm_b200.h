// C ABI of libugemm_b200.so: hand-written sm_100a kernels for the distributed
// GEMM executors (fused stationary GEMM, one-sided tile copy / accumulate,
// zeroing, cross-rank signal barrier) plus the small host runtime they need
// (symmetric allocations over CUDA IPC, TMA descriptor encoding).
//
// Everything here is called from Python through ctypes; all pointers are raw
// device addresses (uint64_t) and every launch takes the cudaStream_t of the
// caller.  The table structs below are filled on the host (numpy structured
// arrays with the same layout) and copied to the device once per cached plan.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// ----------------------------------------------------------------------------
// Tile configuration of the fused GEMM (one CTA, cta_group::1).
// ----------------------------------------------------------------------------
#define UG_BM 128          // rows of one UMMA (and of the small output tile); the large tile has 256 rows
#define UG_BN 256          // output tile cols   (UMMA N, fp32 accumulator = 256 TMEM columns)
#define UG_BK 64           // K elements per pipeline stage (64 bf16 = one 128-byte swizzle row)
#define UG_STAGES 4        // smem ring depth (4 x 48 KiB)
#define UG_MAX_MAPS 4096

// Status codes written to the status word (0 = ok).
#define UG_OK 0
#define UG_ERR_TIMEOUT_MBAR 1      // an mbarrier wait inside the fused kernel ran out
#define UG_ERR_TIMEOUT_FLAG 2      // a staged-chunk flag wait ran out
#define UG_ERR_TIMEOUT_PEER 3      // a cross-rank signal wait ran out (barrier kernel)
#define UG_ERR_BAD_TABLE 4         // a table entry failed an in-kernel bounds check

// One K segment of a task: acc += A[a_row0 + r, a_col0 + k] * B[b_row0 + k, b_col0 + c]
// for k in [0, k_len).  a_map / b_map index the tensor-map table; coordinates are
// in elements of that map.  a_flag / b_flag: first counter index of the staged
// chunks of this operand (one chunk per m tile for A, per n tile for B), -1 when
// the operand is read in place.
typedef struct __attribute__((aligned(16))) {
  int32_t a_map, b_map;
  int32_t a_row0, a_col0;
  int32_t b_row0, b_col0;
  int32_t k_len;
  int32_t a_flag, b_flag;
  int32_t pad[7];
} UgSegment;  // 64 bytes

// One output region C[0:m, 0:n] (+)= sum over segments.
typedef struct __attribute__((aligned(16))) {
  uint64_t c_ptr;        // device address of C(0,0) of this region (may be a peer's memory)
  int64_t ldc;           // elements
  int32_t m, n;
  int32_t seg_begin, seg_count;
  int32_t tile_begin;    // first linear tile index of this task
  int32_t m_tiles, n_tiles;
  int32_t kblocks;       // sum over segments of ceil(k_len / UG_BK)
  int32_t c_mode;        // 0: C += acc (plain read-modify-write), 1: red.add (atomic, any owner), 2: C = acc
  int32_t c_dtype;       // 0: fp32, 1: bf16
  int32_t c_vec;         // 1 when 16-byte accesses to C rows are legal
  int32_t group_m;       // m tiles per raster band (L2 reuse of the A band)
} UgTask;  // 64 bytes

// One piece of a staged copy (claimed by one fetch warp).
typedef struct __attribute__((aligned(16))) {
  uint64_t src, dst;       // byte addresses of the first row
  int64_t src_ld, dst_ld;  // bytes between rows
  int32_t rows;
  int32_t row_bytes;       // payload bytes per row
  int32_t flag;            // counter to bump when the piece has landed
  int32_t mode;            // 0: 16-byte vectors (src 16 B aligned), 1: 2-byte elements (dst aligned, src arbitrary)
} UgPiece;  // 48 bytes

typedef struct {
  uint64_t maps;          // CUtensorMap[num_maps] in device memory (128 B each, 64 B aligned)
  uint64_t tasks;         // UgTask[num_tasks]
  uint64_t segs;          // UgSegment[]
  uint64_t pieces;        // UgPiece[num_pieces]
  uint64_t flags;         // uint32 counters[num_flags] (zero at launch)
  uint64_t flag_need;     // int32 need[num_flags]: pieces that make chunk i complete
  uint64_t piece_counter; // uint32: next piece to claim (zero at launch)
  uint64_t status;        // uint32 status word (first error wins)
  int32_t num_maps, num_tasks, num_pieces, num_flags;
  int32_t total_tiles;
  int32_t tile_m;         // rows per output tile: 128 (0 means 128) or 256
  uint64_t timeout_ns;    // limit of every in-kernel wait
  int32_t num_segs;          // entries of `segs` (for the in-kernel table check)
  int32_t cta_pair;          // 1: tables were lowered for the CTA-pair kernel (ug_fused_gemm_pair)
  uint64_t trace;            // 0 = off; else uint64[grid][trace_slots + 1][UG_TR_FIELDS] timeline records (see UG_TR_*)
  int32_t trace_slots;       // tile iterations recorded per CTA (later ones are dropped)
  int32_t epi_poll_ns;       // pause between the epilogue warps' polls of the accumulator barrier (0 = none)
  uint64_t sched;            // 0 = static round-robin tiles; else uint32[2] {next tile claim, finished workers}, both
                             // zero at launch (the last worker to finish resets them): workers claim tiles dynamically
  int32_t fetch_depth;       // 16-byte loads a fetch-warp lane keeps in flight: 4, 8 or 16 (0 means 16)
  int32_t reserved0;
  uint64_t checksum;         // 0 = off; else a double in device memory to which the kernel adds the sum of all accumulator
                             // values it writes out (one atomic add per epilogue warp and tile); never reset by the kernel
} UgFusedParams;

// Fields of one timeline record (globaltimer nanoseconds unless noted).  Record `trace_slots` of a CTA is
// its summary: UG_TR_S_*.
enum {
  UG_TR_TILE = 0,        // linear tile index + 1
  UG_TR_PROD_BEGIN = 1,  // TMA producer reached the tile
  UG_TR_PROD_FLAGWAIT = 2,  // nanoseconds the producer waited for staged chunks of this tile
  UG_TR_PROD_END = 3,    // last load of the tile issued
  UG_TR_MMA_BEGIN = 4,   // accumulator buffer free, first UMMA may issue (leader CTA only in pair mode)
  UG_TR_MMA_ISSUED = 5,  // last UMMA of the tile issued
  UG_TR_EPI_BEGIN = 6,   // accumulator complete (seen by the first epilogue warp)
  UG_TR_EPI_END = 7,     // first epilogue warp finished its rows
  UG_TR_MMA_CLK = 8,     // clock64() of the SM at UG_TR_MMA_BEGIN
  UG_TR_EPI_CLK = 9,     // clock64() of the SM at UG_TR_EPI_BEGIN: (EPI_CLK - MMA_CLK) / (EPI_BEGIN - MMA_BEGIN) = SM clock
  UG_TR_FIELDS = 16,     // uint64 words per record
  UG_TR_S_START = 0, UG_TR_S_FETCH_END = 1, UG_TR_S_END = 2, UG_TR_S_PIECES = 3,
  UG_TR_S_CLK_START = 4, UG_TR_S_CLK_END = 5   // clock64() of the SM at start / end: SM clock = cycles / nanoseconds
};

// ----------------------------------------------------------------------------
// Host runtime
// ----------------------------------------------------------------------------
int ug_version(void);
// cudaMalloc / cudaFree with the device of the calling thread.
int ug_malloc(uint64_t bytes, uint64_t* out_ptr);
int ug_free(uint64_t ptr);
// Legacy CUDA IPC: 64-byte handles exchanged by the caller (torch.distributed).
int ug_ipc_get_handle(uint64_t ptr, void* handle64);
int ug_ipc_open(const void* handle64, uint64_t* out_ptr);
int ug_ipc_close(uint64_t ptr);
// Encode a 2-D tiled TMA descriptor (row-major matrix, `inner` contiguous).
// dtype: 0 fp32, 1 bf16.  swizzle: 0 none, 3 = 128 B.  Returns the CUresult.
int ug_encode_tensor_map(void* out128, uint64_t base, int dtype, uint64_t inner, uint64_t outer,
                         uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer, int swizzle);
const char* ug_last_error(void);

// ----------------------------------------------------------------------------
// Kernels (all asynchronous on `stream`; return the cudaError_t of the launch)
// ----------------------------------------------------------------------------
// Fused stationary GEMM: persistent tcgen05/TMEM kernel with in-kernel staging
// of remote / misaligned operand slices and local or remote C accumulation.
int ug_fused_gemm(const UgFusedParams* params, int grid, void* stream);
// CTA-pair variant (cta_group::2): a cluster of two CTAs per 256 x 256 tile; `grid` must be even.
int ug_fused_gemm_pair(const UgFusedParams* params, int grid, void* stream);
int ug_fused_gemm_pair_max_pairs(void);
// Dynamic shared memory the fused kernel asks for (for occupancy checks).
int ug_fused_gemm_smem_bytes(void);

// Cross-rank barrier on symmetric counters.  `peer_slots[p]` is the address (in
// this process) of rank p's counter array uint32[world]; the kernel advances the
// local uint32 at `seq_counter`, adds 1 to slot `rank` of every peer and waits until
// its own slots reach the new sequence number.
// Also zeroes `num_clear` uint32 words at `clear_ptr` (plan flags) when non-zero.
int ug_signal_barrier(const uint64_t* peer_slots_dev, int world, int rank, uint64_t seq_counter,
                      uint64_t status, uint64_t timeout_ns, uint64_t clear_ptr, int num_clear,
                      void* stream);
// Point-to-point signals: add `value` to a uint32 counter (possibly in a peer's memory) after all earlier
// work of the stream; wait (bounded) until a local counter has reached `expected`.
int ug_signal_add(uint64_t counter, uint32_t value, void* stream);
int ug_signal_wait(uint64_t counter, uint32_t expected, uint64_t status, uint64_t timeout_ns, void* stream);
// Zero `rows` x `row_bytes` with row pitch `ld_bytes` (16-byte vectors when aligned).
int ug_zero_2d(uint64_t dst, int64_t ld_bytes, int32_t rows, int64_t row_bytes, void* stream);
// dst[r, c] = src[r, c] for a 2-D slice; src may be peer memory.  elem_bytes in {2, 4}.
int ug_pull_2d(uint64_t dst, int64_t dst_ld_bytes, uint64_t src, int64_t src_ld_bytes,
               int32_t rows, int64_t row_bytes, int32_t elem_bytes, void* stream);
// dst[r, c] += src[r, c] with red.add; dst may be peer memory.  dtype: 0 fp32, 1 bf16.
int ug_accumulate_2d(uint64_t dst, int64_t dst_ld_elems, uint64_t src, int64_t src_ld_elems,
                     int32_t rows, int32_t cols, int32_t dtype, void* stream);
// Pack / unpack used by the redistribute path: dst (dense or strided) = cast(src).
// src_dtype / dst_dtype: 0 fp32, 1 bf16.
int ug_convert_2d(uint64_t dst, int64_t dst_ld_elems, int32_t dst_dtype, uint64_t src,
                  int64_t src_ld_elems, int32_t src_dtype, int32_t rows, int32_t cols, void* stream);

#ifdef __cplusplus
}
#endif
