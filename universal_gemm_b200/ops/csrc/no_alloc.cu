// ug_gemm_noalloc: GEMM through the fused tcgen05 kernel with every byte of scratch taken
// from one file-scope device array (see no_alloc.h for who needs this and the rules of use).
//
// Host code below never uses the array's name as an address: the name is only a host-side
// stand-in for the symbol.  The device address is looked up once per device with
// cudaGetSymbolAddress (with that device current) and every address handed to the kernel is
// derived from it.
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include <atomic>
#include <mutex>

#include "no_alloc.h"
#include "ugemm_b200.h"

namespace {

static __device__ __align__(256) unsigned char g_noalloc_scratch[UG_NOALLOC_SCRATCH_BYTES];

// Layout of the table area (bytes from the start of the array).
constexpr uint32_t kOffStatus = 0;          // uint32 status word
constexpr uint32_t kOffMaps = 256;          // 2 x CUtensorMap (128 B each)
constexpr uint32_t kOffTask = 1024;         // 1 x UgTask
constexpr uint32_t kOffSeg = 1280;          // 1 x UgSegment
constexpr uint32_t kOffNeed = 2048;         // int32[UG_NOALLOC_MAX_FLAGS]
constexpr uint32_t kOffFlags = 8192;        // uint32[UG_NOALLOC_MAX_FLAGS + 1] (counters + piece cursor)
constexpr uint32_t kOffPieces = 16384;      // UgPiece[UG_NOALLOC_MAX_PIECES]
static_assert(kOffNeed + 4 * UG_NOALLOC_MAX_FLAGS <= kOffFlags, "need table overlaps counters");
static_assert(kOffFlags + 4 * (UG_NOALLOC_MAX_FLAGS + 1) <= kOffPieces, "counters overlap pieces");
static_assert(kOffPieces + sizeof(UgPiece) * UG_NOALLOC_MAX_PIECES <= UG_NOALLOC_STAGING_OFFSET,
              "piece table overlaps the staging area");

constexpr int kMaxDevices = 64;
// Published with release / read with acquire: a thread that sees a non-zero address also sees the SM count.
std::atomic<uint64_t> g_scratch_addr[kMaxDevices];
int g_num_sms[kMaxDevices] = {};
std::mutex g_setup_mutex;

constexpr int kPieceBytes = 32 * 1024;

inline int64_t round_up(int64_t x, int64_t m) { return (x + m - 1) / m * m; }

int reject(int code, const char* what) {
  fprintf(stderr, "ug_gemm_noalloc: %s\n", what);
  return code;
}

// Once per device, with that device current: resolve the device address of the static array.
int setup_device(int dev) {
  if (g_scratch_addr[dev].load(std::memory_order_acquire) != 0) return 0;
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_scratch_addr[dev].load(std::memory_order_acquire) != 0) return 0;
  unsigned char* ptr = nullptr;
  cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_noalloc_scratch);
  if (e != cudaSuccess || ptr == nullptr) {
    fprintf(stderr, "ug_gemm_noalloc: cudaGetSymbolAddress failed: %s\n", cudaGetErrorString(e));
    return UG_NOALLOC_ERR_SETUP;
  }
  int sms = 0;
  e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (e != cudaSuccess || sms <= 0) return UG_NOALLOC_ERR_SETUP;
  g_num_sms[dev] = sms;
  g_scratch_addr[dev].store(reinterpret_cast<uint64_t>(ptr), std::memory_order_release);
  return 0;
}

struct Operand {
  uint64_t base;
  int64_t ld;      // elements
  int32_t rows, cols;
  bool tma_ok() const { return (base & 15) == 0 && ((ld * 2) & 15) == 0; }
};

// Host images of the tables (static storage: no allocation at call time).
thread_local UgPiece t_pieces[UG_NOALLOC_MAX_PIECES];
thread_local int32_t t_need[UG_NOALLOC_MAX_FLAGS];

}  // namespace

extern "C" int ug_gemm_noalloc(uint64_t a, int64_t lda, uint64_t b, int64_t ldb, uint64_t c, int64_t ldc,
                               int32_t m, int32_t n, int32_t k, int32_t c_dtype, int32_t c_mode,
                               uint64_t status_ptr, void* stream) {
  if (a == 0 || b == 0 || c == 0 || m <= 0 || n <= 0 || k <= 0) return reject(UG_NOALLOC_ERR_INVALID, "null pointer or empty extent");
  if (lda < k || ldb < n || ldc < n) return reject(UG_NOALLOC_ERR_INVALID, "row pitch smaller than the row");
  if ((a & 1) || (b & 1)) return reject(UG_NOALLOC_ERR_INVALID, "A and B must be 2-byte aligned");
  if (c_dtype != 0 && c_dtype != 1) return reject(UG_NOALLOC_ERR_INVALID, "c_dtype must be 0 (fp32) or 1 (bf16)");
  if (c_mode != 0 && c_mode != 2) return reject(UG_NOALLOC_ERR_INVALID, "c_mode must be 0 (add) or 2 (store)");
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (dev < 0 || dev >= kMaxDevices) return reject(UG_NOALLOC_ERR_INVALID, "device index out of range");
  int rc = setup_device(dev);
  if (rc != 0) return rc;
  const uint64_t S = g_scratch_addr[dev].load(std::memory_order_acquire);
  cudaStream_t st = static_cast<cudaStream_t>(stream);

  const Operand A{a, lda, m, k}, B{b, ldb, k, n};
  const bool stage_a = !A.tma_ok(), stage_b = !B.tma_ok();
  const int m_tiles = (m + UG_BM - 1) / UG_BM, n_tiles = (n + UG_BN - 1) / UG_BN;

  // Staging layout and size check against the static array.
  const int64_t a_ld_s = round_up(k, 64), b_ld_s = round_up(n, 64);
  const int64_t a_bytes = stage_a ? round_up(static_cast<int64_t>(m) * a_ld_s * 2, 1024) : 0;
  const int64_t b_bytes = stage_b ? round_up(static_cast<int64_t>(k) * b_ld_s * 2, 1024) : 0;
  const int num_flags = (stage_a ? m_tiles : 0) + (stage_b ? n_tiles : 0);
  if (a_bytes + b_bytes > static_cast<int64_t>(UG_NOALLOC_STAGING_BYTES) || num_flags > UG_NOALLOC_MAX_FLAGS) {
    fprintf(stderr,
            "ug_gemm_noalloc: m=%d n=%d k=%d needs %lld bytes of staging and %d chunk counters; the static "
            "scratch array offers %u bytes and %d counters\n",
            m, n, k, static_cast<long long>(a_bytes + b_bytes), num_flags, UG_NOALLOC_STAGING_BYTES,
            UG_NOALLOC_MAX_FLAGS);
    return UG_NOALLOC_ERR_TOO_LARGE;
  }
  const uint64_t a_stage = S + UG_NOALLOC_STAGING_OFFSET, b_stage = a_stage + a_bytes;

  // Pieces of the staged copies (A: chunks of UG_BM rows, B: chunks of UG_BN columns).
  int num_pieces = 0;
  const int a_flag0 = 0, b_flag0 = stage_a ? m_tiles : 0;
  auto add_pieces = [&](const Operand& op, bool is_a, uint64_t dst_base, int64_t dst_ld, int flag0) -> bool {
    const bool vec = (op.base & 15) == 0 && ((op.ld * 2) & 15) == 0;
    const int chunks = is_a ? m_tiles : n_tiles;
    for (int ch = 0; ch < chunks; ++ch) {
      const int r0 = is_a ? ch * UG_BM : 0, r1 = is_a ? (op.rows < (ch + 1) * UG_BM ? op.rows : (ch + 1) * UG_BM) : op.rows;
      const int c0 = is_a ? 0 : ch * UG_BN, c1 = is_a ? op.cols : (op.cols < (ch + 1) * UG_BN ? op.cols : (ch + 1) * UG_BN);
      const int row_bytes = (c1 - c0) * 2;
      int rpp = kPieceBytes / (row_bytes > 0 ? row_bytes : 1);
      if (rpp < 1) rpp = 1;
      int count = 0;
      for (int r = r0; r < r1; r += rpp) {
        if (num_pieces >= UG_NOALLOC_MAX_PIECES) return false;
        UgPiece& p = t_pieces[num_pieces++];
        p.src = op.base + (static_cast<int64_t>(r) * op.ld + c0) * 2;
        p.dst = dst_base + (static_cast<int64_t>(r) * dst_ld + c0) * 2;
        p.src_ld = op.ld * 2;
        p.dst_ld = dst_ld * 2;
        p.rows = (r1 - r) < rpp ? (r1 - r) : rpp;
        p.row_bytes = row_bytes;
        p.flag = flag0 + ch;
        p.mode = vec ? 0 : 1;
        ++count;
      }
      t_need[flag0 + ch] = count;
    }
    return true;
  };
  if (stage_a && !add_pieces(A, true, a_stage, a_ld_s, a_flag0)) return reject(UG_NOALLOC_ERR_TOO_LARGE, "too many copy pieces for the static piece table");
  if (stage_b && !add_pieces(B, false, b_stage, b_ld_s, b_flag0)) return reject(UG_NOALLOC_ERR_TOO_LARGE, "too many copy pieces for the static piece table");

  // TMA descriptors: A (k inner, m outer, box 64 x 128), B (n inner, k outer, box 64 x 64).
  alignas(64) unsigned char maps[256];
  rc = ug_encode_tensor_map(maps, stage_a ? a_stage : a, 1, static_cast<uint64_t>(k), static_cast<uint64_t>(m),
                            static_cast<uint64_t>((stage_a ? a_ld_s : lda) * 2), UG_BK, UG_BM, 3);
  if (rc != 0) return reject(UG_NOALLOC_ERR_SETUP, "TMA descriptor of A could not be encoded");
  rc = ug_encode_tensor_map(maps + 128, stage_b ? b_stage : b, 1, static_cast<uint64_t>(n), static_cast<uint64_t>(k),
                            static_cast<uint64_t>((stage_b ? b_ld_s : ldb) * 2), 64, UG_BK, 3);
  if (rc != 0) return reject(UG_NOALLOC_ERR_SETUP, "TMA descriptor of B could not be encoded");

  UgSegment seg;
  memset(&seg, 0, sizeof(seg));
  seg.a_map = 0;
  seg.b_map = 1;
  seg.k_len = k;
  seg.a_flag = stage_a ? a_flag0 : -1;
  seg.b_flag = stage_b ? b_flag0 : -1;
  UgTask task;
  memset(&task, 0, sizeof(task));
  const int c_elem = c_dtype == 0 ? 4 : 2;
  task.c_ptr = c;
  task.ldc = ldc;
  task.m = m;
  task.n = n;
  task.seg_begin = 0;
  task.seg_count = 1;
  task.tile_begin = 0;
  task.m_tiles = m_tiles;
  task.n_tiles = n_tiles;
  task.kblocks = (k + UG_BK - 1) / UG_BK;
  task.c_mode = c_mode;
  task.c_dtype = c_dtype;
  task.c_vec = ((c & 15) == 0 && ((ldc * c_elem) & 15) == 0) ? 1 : 0;
  task.group_m = m_tiles <= 16 ? m_tiles : 16;

  // Upload the tables and clear what must start at zero (status word, counters, piece cursor).
#define UG_TRY(call)                                  \
  do {                                                \
    cudaError_t err__ = (call);                       \
    if (err__ != cudaSuccess) return static_cast<int>(err__); \
  } while (0)
  UG_TRY(cudaMemsetAsync(reinterpret_cast<void*>(S + kOffStatus), 0, 256, st));
  UG_TRY(cudaMemsetAsync(reinterpret_cast<void*>(S + kOffFlags), 0, 4 * (UG_NOALLOC_MAX_FLAGS + 1), st));
  UG_TRY(cudaMemcpyAsync(reinterpret_cast<void*>(S + kOffMaps), maps, 256, cudaMemcpyHostToDevice, st));
  UG_TRY(cudaMemcpyAsync(reinterpret_cast<void*>(S + kOffTask), &task, sizeof(task), cudaMemcpyHostToDevice, st));
  UG_TRY(cudaMemcpyAsync(reinterpret_cast<void*>(S + kOffSeg), &seg, sizeof(seg), cudaMemcpyHostToDevice, st));
  if (num_flags > 0)
    UG_TRY(cudaMemcpyAsync(reinterpret_cast<void*>(S + kOffNeed), t_need, 4 * num_flags, cudaMemcpyHostToDevice, st));
  if (num_pieces > 0)
    UG_TRY(cudaMemcpyAsync(reinterpret_cast<void*>(S + kOffPieces), t_pieces, sizeof(UgPiece) * num_pieces,
                           cudaMemcpyHostToDevice, st));
#undef UG_TRY

  UgFusedParams P;
  memset(&P, 0, sizeof(P));
  P.maps = S + kOffMaps;
  P.tasks = S + kOffTask;
  P.segs = S + kOffSeg;
  P.pieces = S + kOffPieces;
  P.flags = S + kOffFlags;
  P.flag_need = S + kOffNeed;
  P.piece_counter = S + kOffFlags + 4ull * num_flags;
  P.status = status_ptr != 0 ? status_ptr : S + kOffStatus;
  P.num_maps = 2;
  P.num_tasks = 1;
  P.num_segs = 1;
  P.num_pieces = num_pieces;
  P.num_flags = num_flags;
  P.total_tiles = m_tiles * n_tiles;
  P.timeout_ns = 2000000000ull;
  const int sms = g_num_sms[dev];
  const int grid = (num_pieces > 0 || P.total_tiles >= sms) ? sms : P.total_tiles;
  return ug_fused_gemm(&P, grid, stream);
}
