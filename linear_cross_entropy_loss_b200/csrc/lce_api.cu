// C ABI of the library (declared in include/lce_b200.h): argument validation, workspace layout,
// TMA tensor-map construction and kernel launches. No device memory is allocated here.
#include "../../include/lce_b200.h"

#include "aux_kernels.cuh"
#include "gemm_sm100.cuh"
#include "peer_exchange.cuh"

#include <algorithm>
#include <atomic>
#include <cstddef>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

namespace {

using namespace lce;

std::atomic<long long> g_launches{0};

// ------------------------------------------------------------------------------------------------
// device bookkeeping
// ------------------------------------------------------------------------------------------------
constexpr int kMaxDevices = 64;
std::mutex g_mutex;
bool g_device_ready[kMaxDevices] = {};
int g_device_sms[kMaxDevices] = {};

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;

template <int kKind, bool kAMN, bool kBMN, int kEpi, bool kMon>
cudaError_t set_smem_attr() {
  cudaError_t e = cudaFuncSetAttribute(lce_gemm_kernel<kKind, kAMN, kBMN, kEpi, kMon>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kGemmSmemBytes);
  if (e != cudaSuccess) return e;
  return cudaFuncSetAttribute(lce_gemm_pair_kernel<kKind, kAMN, kBMN, kEpi, kMon>,
                              cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kGemmPairSmemBytes);
}

template <int kKind>
cudaError_t set_smem_attr_kind() {
  cudaError_t e;
  if ((e = set_smem_attr<kKind, false, true, EPI_FWD, false>()) != cudaSuccess) return e;
  if ((e = set_smem_attr<kKind, false, true, EPI_FWD, true>()) != cudaSuccess) return e;
  if ((e = set_smem_attr<kKind, false, false, EPI_F32, false>()) != cudaSuccess) return e;
  if ((e = set_smem_attr<kKind, true, true, EPI_F32, false>()) != cudaSuccess) return e;
  if ((e = set_smem_attr<kKind, false, true, EPI_F32, false>()) != cudaSuccess) return e;
  if ((e = set_smem_attr<kKind, true, false, EPI_F32, false>()) != cudaSuccess) return e;
  return cudaSuccess;
}

// Once per device: check the architecture, raise the dynamic shared-memory limit of every GEMM
// instantiation, fetch the tensor-map encoder from the driver. Returns the SM count through *sms.
int ensure_device(int* sms) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return LCE_ERR_CUDA;
  if (dev < 0 || dev >= kMaxDevices) return LCE_ERR_UNSUPPORTED_DEVICE;
  std::lock_guard<std::mutex> lock(g_mutex);
  if (!g_device_ready[dev]) {
    int major = 0, count = 0;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) return LCE_ERR_CUDA;
    if (cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return LCE_ERR_CUDA;
    if (major != 10) return LCE_ERR_UNSUPPORTED_DEVICE;
    if (set_smem_attr_kind<KIND_F16>() != cudaSuccess) return LCE_ERR_CUDA;
    if (set_smem_attr_kind<KIND_BF16>() != cudaSuccess) return LCE_ERR_CUDA;
    if (set_smem_attr_kind<KIND_TF32>() != cudaSuccess) return LCE_ERR_CUDA;
    if (g_encode == nullptr) {
      void* fn = nullptr;
      cudaDriverEntryPointQueryResult qres;
      if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess ||
          qres != cudaDriverEntryPointSuccess || fn == nullptr)
        return LCE_ERR_DRIVER;
      g_encode = reinterpret_cast<EncodeTiledFn>(fn);
    }
    g_device_sms[dev] = count;
    g_device_ready[dev] = true;
  }
  *sms = g_device_sms[dev];
  return LCE_OK;
}

int sm_count_or_default() {
  int dev = 0, count = 0;
  if (cudaGetDevice(&dev) == cudaSuccess &&
      cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && count > 0)
    return count;
  return 148;  // B200
}

// ------------------------------------------------------------------------------------------------
// shapes, workspace
// ------------------------------------------------------------------------------------------------
inline int elem_size(int dtype) { return dtype == LCE_DTYPE_F32 ? 4 : 2; }
inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }
inline long long round_up(long long v, long long a) { return (v + a - 1) / a * a; }
// Tiles are 128 rows x 256 columns; sizes that are not multiples are padded inside the workspace and masked in
// the kernels (TMA zero-fills what it reads outside x, W).
inline long long vocab_pad(const lce_problem* p) { return round_up(p->vocab_local, BLOCK_N); }
inline long long hidden_pad(const lce_problem* p) { return round_up(p->hidden, BLOCK_N); }

int validate_problem(const lce_problem* p) {
  if (p == nullptr) return LCE_ERR_INVALID_ARGUMENT;
  if (p->dtype != LCE_DTYPE_F16 && p->dtype != LCE_DTYPE_BF16 && p->dtype != LCE_DTYPE_F32)
    return LCE_ERR_INVALID_ARGUMENT;
  if (p->n_rows_total <= 0 || p->chunk_rows <= 0 || p->hidden <= 0 || p->vocab_local <= 0)
    return LCE_ERR_INVALID_ARGUMENT;
  if (p->world < 1 || p->vocab_offset < 0) return LCE_ERR_INVALID_ARGUMENT;
  if ((p->slab_mode != LCE_SLAB_DEFAULT && p->slab_mode != LCE_SLAB_PER_TILE) || p->chunk_buffers < 0 ||
      p->chunk_buffers > 2)
    return LCE_ERR_INVALID_ARGUMENT;
  if (!(p->logit_scale > 0.f) || !(p->z_regularization >= 0.f)) return LCE_ERR_INVALID_ARGUMENT;
  if (p->chunk_rows % BLOCK_M != 0) return LCE_ERR_UNSUPPORTED_SHAPE;
  // rows of x are handled 8 elements at a time. The vocabulary may have any size: columns past it are masked in
  // every epilogue; only the ROWS of W and dW must start on 16-byte boundaries (checked where they are used).
  if (p->hidden % 8 != 0) return LCE_ERR_UNSUPPORTED_SHAPE;
  // TMA coordinates and the kernels' tile counters are 32-bit
  if (p->n_rows_total > (1ll << 30) || p->hidden > (1ll << 30) || p->vocab_local > (1ll << 30))
    return LCE_ERR_TOO_LARGE;
  return LCE_OK;
}

// K-split of the dx contraction (K = vocab_local). More splits fill the SMs in whole waves (128 tiles on 74 CTA pairs
// are 1.73 waves; four times as many units are 6.92) but cost fp32 partials that a second kernel has to sum; one
// split lets the contraction write dx itself. The choice minimises a small cost model: contraction time at the wave
// efficiency of the split + time of the partial traffic (rates measured on B200: 1.3 PFLOP/s, 4.5 TB/s).
int choose_dx_splits(const lce_problem* p, int sms) {
  const long long tiles = (p->chunk_rows / BLOCK_M) * (hidden_pad(p) / BLOCK_N);
  const long long kblocks = vocab_pad(p) * elem_size(p->dtype) / 128;
  const double gemm_us = 2.0 * (double)p->chunk_rows * (double)hidden_pad(p) * (double)vocab_pad(p) / 1.3e9;
  const double row_elems = (double)p->chunk_rows * (double)hidden_pad(p);
  int best = 1;
  double best_us = 0.0;
  for (int s = 1; s <= 16; s *= 2) {
    if (kblocks % s != 0 || (s > 1 && kblocks / s < 8)) break;
    const long long units = tiles * s;
    const long long waves = (units + sms - 1) / sms;
    const double eff = (double)units / (double)(waves * sms);
    // the reduction reads s fp32 partials and writes the result once, plus a launch and its gap; the partial
    // stores overlap the contraction and are charged at half their traffic (they cost energy more than time)
    const double extra_us = s == 1 ? 0.0 : row_elems * (6.0 * s + 2.0) / 4.5e6 + 4.0;
    const double us = gemm_us / eff + extra_us;
    if (s == 1 || us < best_us) {
      best_us = us;
      best = s;
    }
  }
  return best;
}

struct Workspace {
  PassScalars* scalars;
  float* tile_max;
  float* tile_sum;
  float* tile_ez;
  float* tile_sq;
  float* target_logit;
  float* lse;
  float* row_ref;   // row-reference mode: row max of the first forward = reference of a conditional re-run
  float* row_base;  // row-reference mode: the reference the row's slab and sums were computed with
  float* row_coef;  // row-reference mode: exp(base - lse) (1 + 2 z_reg lse), 0 for ignored rows
  int* rescue_groups;  // row-reference mode: one flag per 256 rows of the chunk: forward must be re-run for them
  int* rescue_flag;    //   ... and the word after them: some group of the chunk is flagged
  int n_rescue;        //   number of ints in rescue_groups, the flag word included
  void* slab;
  void* xs;         // row-reference mode: row_coef[i] * x[i, :] for the rows of the chunk
  float* dx_part;
  int dx_splits;
  size_t total;
};

// fp16 slabs hold exp(z - tile max) and are rescaled in a separate pass; bf16 / fp32 slabs hold
// exp(z - row reference) and feed the gradient GEMMs directly (see gemm_sm100.cuh).
inline bool row_reference_mode(const lce_problem* p) {
  return p->dtype != LCE_DTYPE_F16 && p->slab_mode != LCE_SLAB_PER_TILE;
}

inline int chunk_buffer_count(const lce_problem* p) { return p->chunk_buffers == 2 ? 2 : 1; }
// The set of per-chunk buffers the chunk that contains row0 uses: consecutive chunks alternate.
inline int chunk_buffer_of(const lce_problem* p, long long row0) {
  return (int)((row0 / p->chunk_rows) % chunk_buffer_count(p));
}

// Workspace: pass accumulators | per-chunk buffers (one or two sets; `buf` selects the one returned) | dx partials.
Workspace layout_workspace(const lce_problem* p, void* base, int sms, int buf = 0) {
  Workspace w;
  const size_t n_tiles = (size_t)(vocab_pad(p) / BLOCK_N);
  const size_t rows = (size_t)p->chunk_rows;
  const size_t stat_bytes = align_up(n_tiles * rows * sizeof(float), 256);
  char* b = reinterpret_cast<char*>(base);
  size_t off = 0;
  auto take = [&](size_t bytes) {
    char* ptr = b + off;
    off += align_up(bytes, 256);
    return ptr;
  };
  w.scalars = reinterpret_cast<PassScalars*>(take(sizeof(PassScalars)));
  for (int k = 0; k < chunk_buffer_count(p); ++k) {
    Workspace t = w;
    t.tile_max = reinterpret_cast<float*>(take(stat_bytes));
    t.tile_sum = reinterpret_cast<float*>(take(stat_bytes));
    t.tile_ez = reinterpret_cast<float*>(take(p->monitoring ? stat_bytes : 0));
    t.tile_sq = reinterpret_cast<float*>(take(p->monitoring ? stat_bytes : 0));
    t.target_logit = reinterpret_cast<float*>(take(rows * sizeof(float)));
    t.lse = reinterpret_cast<float*>(take(rows * sizeof(float)));
    t.row_ref = reinterpret_cast<float*>(take(rows * sizeof(float)));
    t.row_base = reinterpret_cast<float*>(take(rows * sizeof(float)));
    t.row_coef = reinterpret_cast<float*>(take(rows * sizeof(float)));
    // group index of a row is (chunk-local row) / 256 <= rows / 256; one more word holds the chunk's flag
    t.n_rescue = (int)(rows / 256 + 2);
    t.rescue_groups = reinterpret_cast<int*>(take((size_t)t.n_rescue * sizeof(int)));
    t.rescue_flag = t.rescue_groups + (t.n_rescue - 1);
    if (p->want_grad) {
      t.slab = take(rows * (size_t)vocab_pad(p) * elem_size(p->dtype));
      t.xs = row_reference_mode(p) ? take(rows * (size_t)hidden_pad(p) * elem_size(p->dtype)) : nullptr;
    } else {
      t.slab = nullptr;
      t.xs = nullptr;
    }
    if (k == buf) w = t;
  }
  w.dx_splits = choose_dx_splits(p, sms);
  w.dx_part = p->want_grad
                  ? reinterpret_cast<float*>(take((size_t)w.dx_splits * rows * (size_t)hidden_pad(p) * sizeof(float)))
                  : nullptr;
  w.total = off;
  return w;
}

// ------------------------------------------------------------------------------------------------
// tensor maps
// ------------------------------------------------------------------------------------------------
// 2-D row-major tensor [outer, inner] (inner contiguous, rows `ld` elements apart), 128-byte swizzle.
int make_tmap(CUtensorMap* map, int dtype, const void* base, long long inner, long long outer, long long ld,
              int box_inner, int box_outer, bool atom32) {
  const int es = elem_size(dtype);
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0 || ((ld * es) & 15) != 0) return LCE_ERR_MISALIGNED;
  if (box_inner * es != 128 || box_outer > 256 || box_outer < 1) return LCE_ERR_INVALID_ARGUMENT;
  const CUtensorMapDataType dt = dtype == LCE_DTYPE_F16    ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                 : dtype == LCE_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                           : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  const cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)outer};
  const cuuint64_t strides[1] = {(cuuint64_t)(ld * es)};
  const cuuint32_t box[2] = {(cuuint32_t)box_inner, (cuuint32_t)box_outer};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = g_encode(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr,
                              CU_TENSOR_MAP_INTERLEAVE_NONE,
                              atom32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? LCE_OK : LCE_ERR_DRIVER;
}

// Operand tile boxes: K-major operand -> one box (128 bytes of K) x (tile rows);
//                     MN-major operand -> boxes of (128 bytes of MN) x (BLOCK_K rows of K).
int make_operand_tmap(CUtensorMap* map, int dtype, bool mn_major, const void* base, long long inner,
                      long long outer, long long ld, int tile_mn) {
  const int per128 = 128 / elem_size(dtype);
  // MN-major 32-bit operands need the 32-byte-atom swizzle (see make_smem_desc)
  return mn_major ? make_tmap(map, dtype, base, inner, outer, ld, per128, per128, dtype == LCE_DTYPE_F32)
                  : make_tmap(map, dtype, base, inner, outer, ld, per128, tile_mn, false);
}

// Output tile map for the epilogues' TMA stores: boxes of 32 rows x 128 bytes of a row-major [outer, inner] tensor.
int make_store_tmap(CUtensorMap* map, int dtype, const void* base, long long inner, long long outer, long long ld) {
  return make_tmap(map, dtype, base, inner, outer, ld, 128 / elem_size(dtype), 32, false);
}

// LCE_EPILOGUE_STORE=direct (read once, at the first launch) keeps the epilogues on per-thread global stores
// instead of shared-memory staging + TMA; for A/B measurements of the two forms.
bool epilogue_tma_enabled() {
  static const bool on = [] {
    const char* v = std::getenv("LCE_EPILOGUE_STORE");
    return !(v != nullptr && std::strcmp(v, "direct") == 0);
  }();
  return on;
}

// LCE_RASTER_GROUP (A/B measurements; read once per process): unset or "auto" lets choose_raster_group decide,
// "0" walks every tile grid without bands, a positive number forces bands of that many tiles.
int raster_group_override() {
  static const int value = [] {
    const char* v = std::getenv("LCE_RASTER_GROUP");
    if (v == nullptr || *v == 0 || std::strcmp(v, "auto") == 0) return -2;
    char* end = nullptr;
    const long g = std::strtol(v, &end, 10);
    if (end == v || g < 0 || g > (1 << 20)) return -2;
    return g == 0 ? -1 : (int)g;
  }();
  return value;
}

// Bands for the walk over the tile grid (unit_to_tile); 0 = none. `fast_tiles` tiles of `fast_tile_rows` rows or
// columns lie along the dimension that consecutive units walk first. A grid longer than 4096 rows (16 tiles of
// the CTA-pair kernel) along that dimension is walked in equal bands of at most 4096 rows: the tiles in flight
// then form the same 16 x 4.6 block as at the default chunk of 4096 rows, and less of the long operand is fetched
// from DRAM again (forward at 8192 rows x 8192 hidden x 16384 columns, ncu: 2.5 GB read instead of 5.1 GB, of
// 0.4 GB that exist). Measured on two B200s inside the power-capped step, TFLOP/s of the whole step without bands
// / with bands of 8, 11, 16, 24 tiles (all three contractions have 32-tile grids in both shapes):
//   N=131072 H=8192 V=262144 chunk 8192:  1054 / 1058, 1060, 1097, 1055    (bands of 4: 1022)
//   N=65536  H=4096 V=131072 chunk 8192:  1211 / 1230, 1205, 1239, 1225
// and the default shape (16-tile grids) with its forward cut into two bands of 8: 1236 against 1247. Why exactly
// 16 wins is not understood (narrower bands fetch even fewer bytes); the rule keeps what was measured.
int choose_raster_group(int fast_tiles, int fast_tile_rows) {
  const int widest = 4096 / fast_tile_rows;  // 16 tiles of 256, 32 of 128
  if (fast_tiles <= widest) return 0;
  const int bands = (fast_tiles + widest - 1) / widest;
  return (fast_tiles + bands - 1) / bands;  // equal bands rather than a narrow last one
}

// ------------------------------------------------------------------------------------------------
// launches
// ------------------------------------------------------------------------------------------------
int check_launch() {
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return cudaGetLastError() == cudaSuccess ? LCE_OK : LCE_ERR_CUDA;
}

// Optional per-launch timing of the three tensor-core contractions (lce_profile_enable): a CUDA event
// pair is recorded on the launching stream around each GEMM kernel and read back by lce_profile_read.
enum : int { PROF_FWD = 0, PROF_DX = 1, PROF_DW = 2, PROF_KINDS = 3 };
struct ProfSpan {
  cudaEvent_t start, stop;
  int kind;
};
std::mutex g_prof_mutex;
bool g_prof_enabled = false;
std::vector<ProfSpan> g_prof_spans;      // recorded since the last read
std::vector<ProfSpan> g_prof_free;       // event pairs ready for reuse

struct ProfScope {
  cudaStream_t st;
  ProfSpan span;
  bool active = false;
  ProfScope(int kind, cudaStream_t stream) : st(stream) {
    std::lock_guard<std::mutex> lock(g_prof_mutex);
    if (!g_prof_enabled) return;
    if (!g_prof_free.empty()) {
      span = g_prof_free.back();
      g_prof_free.pop_back();
    } else if (cudaEventCreate(&span.start) != cudaSuccess || cudaEventCreate(&span.stop) != cudaSuccess) {
      return;
    }
    span.kind = kind;
    active = cudaEventRecord(span.start, st) == cudaSuccess;
  }
  ~ProfScope() {
    if (!active) return;
    cudaEventRecord(span.stop, st);
    std::lock_guard<std::mutex> lock(g_prof_mutex);
    g_prof_spans.push_back(span);
  }
};

// With an even number of 128-row tiles (and at least two SMs) a contraction runs on the CTA-pair kernel:
// 256 x 256 tiles, one per cluster of two CTAs, each CTA loading 128 rows of A and 128 of the 256 B columns.
// The B tensor map must be built for the variant that will run (rows_of_b_tile).
bool use_pair_kernel(long long m_tiles128, int sms) { return (m_tiles128 % 2 == 0) && sms >= 2; }
int rows_of_b_tile(bool pair) { return pair ? BLOCK_N / 2 : BLOCK_N; }

// gp.m_tiles counts 128-row tiles; `pair` must be the value the tensor maps were built for.
template <int kKind, bool kAMN, bool kBMN, int kEpi, bool kMon>
int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const GemmParams& gp_in, int sms,
                cudaStream_t st, bool pair) {
  GemmParams gp = gp_in;
  if (pair && gp.m_tiles % 2 != 0) return LCE_ERR_INVALID_ARGUMENT;
  if (pair) gp.m_tiles /= 2;
  const long long units = (long long)gp.splits * gp.n_tiles * gp.m_tiles;
  if (units <= 0 || units > (1ll << 30)) return LCE_ERR_TOO_LARGE;
  {
    // 0: what LCE_RASTER_GROUP says (from the shape unless set), -1: none, -2: from the shape, > 0: as given
    int want = gp.raster_group;
    if (want == 0) want = raster_group_override();
    if (want == -2)
      want = gp.n_fastest ? choose_raster_group(gp.n_tiles, BLOCK_N)
                          : choose_raster_group(gp.m_tiles, pair ? 2 * BLOCK_M : BLOCK_M);
    gp.raster_group = want > 0 ? want : 0;
  }
  if (pair) {
    const long long clusters = units < sms / 2 ? units : sms / 2;
    lce_gemm_pair_kernel<kKind, kAMN, kBMN, kEpi, kMon>
        <<<(int)(2 * clusters), kGemmThreads, kGemmPairSmemBytes, st>>>(ta, tb, tc, gp);
  } else {
    const int grid = (int)(units < sms ? units : sms);
    lce_gemm_kernel<kKind, kAMN, kBMN, kEpi, kMon><<<grid, kGemmThreads, kGemmSmemBytes, st>>>(ta, tb, tc, gp);
  }
  return check_launch();
}

template <bool kAMN, bool kBMN, int kEpi, bool kMon>
int launch_gemm_dtype(int dtype, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc,
                      const GemmParams& gp, int sms, cudaStream_t st, bool pair) {
  switch (dtype) {
    case LCE_DTYPE_F16: return launch_gemm<KIND_F16, kAMN, kBMN, kEpi, kMon>(ta, tb, tc, gp, sms, st, pair);
    case LCE_DTYPE_BF16: return launch_gemm<KIND_BF16, kAMN, kBMN, kEpi, kMon>(ta, tb, tc, gp, sms, st, pair);
    case LCE_DTYPE_F32: return launch_gemm<KIND_TF32, kAMN, kBMN, kEpi, kMon>(ta, tb, tc, gp, sms, st, pair);
  }
  return LCE_ERR_INVALID_ARGUMENT;
}

// Rows [row0, row0 + rows) must lie inside ONE chunk (chunks start at multiples of chunk_rows); a call may
// cover a whole chunk or a 128-aligned part of it.
int check_chunk(const lce_problem* p, int64_t row0, int64_t rows) {
  if (row0 < 0 || rows <= 0 || rows > p->chunk_rows || row0 + rows > p->n_rows_total) return LCE_ERR_INVALID_ARGUMENT;
  if (row0 % p->chunk_rows + round_up(rows, BLOCK_M) > p->chunk_rows) return LCE_ERR_INVALID_ARGUMENT;
  if (row0 % BLOCK_M != 0) return LCE_ERR_UNSUPPORTED_SHAPE;
  // only the last rows of the whole problem may leave a 128-row tile partly empty
  if (rows % BLOCK_M != 0 && row0 + rows != p->n_rows_total) return LCE_ERR_UNSUPPORTED_SHAPE;
  return LCE_OK;
}

inline int grid_for(long long items, int per_block, int sms, int waves) {
  long long g = (items + per_block - 1) / per_block;
  const long long cap = (long long)sms * waves;
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  return (int)g;
}

}  // namespace

// ================================================================================================
// exported entry points
// ================================================================================================
extern "C" {

int lce_version(void) { return 100; }

const char* lce_status_string(int status) {
  switch (status) {
    case LCE_OK: return "ok";
    case LCE_ERR_INVALID_ARGUMENT: return "invalid argument";
    case LCE_ERR_UNSUPPORTED_SHAPE:
      return "unsupported shape (chunk rows % 128 and hidden % 8 must be 0; calls start on 128-row boundaries)";
    case LCE_ERR_MISALIGNED: return "pointer or row stride not 16-byte aligned";
    case LCE_ERR_UNSUPPORTED_DEVICE: return "device is not compute capability 10.x (sm_100a required)";
    case LCE_ERR_CUDA: return "CUDA runtime error";
    case LCE_ERR_DEVICE_TIMEOUT: return "a bounded in-kernel wait ran out (device status word set)";
    case LCE_ERR_DRIVER: return "driver call failed (cuTensorMapEncodeTiled)";
    case LCE_ERR_TOO_LARGE: return "size exceeds the supported maximum";
  }
  return "unknown status";
}

long long lce_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int lce_workspace_bytes(const lce_problem* p, size_t* bytes) {
  const int v = validate_problem(p);
  if (v != LCE_OK) return v;
  if (bytes == nullptr) return LCE_ERR_INVALID_ARGUMENT;
  *bytes = layout_workspace(p, nullptr, sm_count_or_default()).total;
  return LCE_OK;
}

int lce_begin(const lce_problem* p, const int64_t* labels, void* workspace, void* stream) {
  int v = validate_problem(p);
  if (v != LCE_OK) return v;
  if (labels == nullptr || workspace == nullptr) return LCE_ERR_INVALID_ARGUMENT;
  int sms = 0;
  if ((v = ensure_device(&sms)) != LCE_OK) return v;
  const Workspace w = layout_workspace(p, workspace, sms, 0);
  int* groups2 = chunk_buffer_count(p) == 2 ? layout_workspace(p, workspace, sms, 1).rescue_groups : nullptr;
  begin_kernel<<<1, 1024, 0, (cudaStream_t)stream>>>(reinterpret_cast<const long long*>(labels),
                                                     (long long)p->n_rows_total, (long long)p->ignore_index,
                                                     w.scalars, w.rescue_groups, groups2, w.n_rescue);
  return check_launch();
}

int lce_forward_chunk(const lce_problem* p, const void* x, int64_t x_ld, const void* weight, int64_t w_ld,
                      const int64_t* labels, int64_t row0, int64_t rows, void* workspace, float* row_parts_local,
                      void* stream) {
  int v = validate_problem(p);
  if (v != LCE_OK) return v;
  if ((v = check_chunk(p, row0, rows)) != LCE_OK) return v;
  if (!x || !weight || !labels || !workspace || !row_parts_local) return LCE_ERR_INVALID_ARGUMENT;
  if (x_ld < p->hidden || w_ld < p->vocab_local) return LCE_ERR_INVALID_ARGUMENT;
  int sms = 0;
  if ((v = ensure_device(&sms)) != LCE_OK) return v;
  cudaStream_t st = (cudaStream_t)stream;
  const Workspace w = layout_workspace(p, workspace, sms, chunk_buffer_of(p, row0));
  const int es = elem_size(p->dtype);
  const long long local0 = row0 % p->chunk_rows;  // first row inside the chunk's slab and statistics

  const long long rows_pad = round_up(rows, BLOCK_M);
  const long long v_pad = vocab_pad(p);
  const bool pair = use_pair_kernel(rows_pad / BLOCK_M, sms);
  CUtensorMap ta, tb;
  if ((v = make_operand_tmap(&ta, p->dtype, false, x, p->hidden, p->n_rows_total, x_ld, BLOCK_M)) != LCE_OK) return v;
  if ((v = make_operand_tmap(&tb, p->dtype, true, weight, p->vocab_local, p->hidden, w_ld, rows_of_b_tile(pair))) !=
      LCE_OK)
    return v;

  GemmParams gp;
  memset(&gp, 0, sizeof(gp));
  // the slab leaves the epilogue through shared memory and TMA stores: whole 128-byte lines instead of one 32-byte
  // sector per thread and instruction
  CUtensorMap tc = ta;
  if (p->want_grad && w.slab != nullptr && epilogue_tma_enabled()) {
    if ((v = make_store_tmap(&tc, p->dtype, w.slab, v_pad, p->chunk_rows, v_pad)) != LCE_OK) return v;
    gp.out_tma = 1;
    gp.c_row0 = (int)local0;
  }
  gp.m_tiles = (int)(rows_pad / BLOCK_M);
  gp.n_tiles = (int)(v_pad / BLOCK_N);
  gp.splits = 1;
  gp.k_blocks = (int)((p->hidden * es + 127) / 128);
  gp.a_mn0 = (int)row0;
  gp.slab = w.slab ? reinterpret_cast<char*>(w.slab) + (size_t)local0 * (size_t)v_pad * es : nullptr;
  gp.slab_ld = v_pad;
  gp.rows_valid = (int)rows;
  gp.cols_valid = (int)p->vocab_local;
  gp.store_slab = (p->want_grad && w.slab != nullptr) ? 1 : 0;
  gp.tile_mode = row_reference_mode(p) ? 0 : 1;
  gp.tile_max = w.tile_max + local0;
  gp.tile_sum = w.tile_sum + local0;
  gp.tile_ez = w.tile_ez + local0;
  gp.tile_sq = w.tile_sq + local0;
  gp.stat_ld = p->chunk_rows;
  gp.target_logit = w.target_logit + local0;
  gp.labels = reinterpret_cast<const long long*>(labels) + row0;
  gp.ignore_index = p->ignore_index;
  gp.vocab_offset = p->vocab_offset;
  gp.scale = p->logit_scale;
  gp.status = &w.scalars->status;

  const int blocks = (int)((rows + 31) / 32);
  const long long* lab = reinterpret_cast<const long long*>(labels) + row0;
  float* parts = row_parts_local + local0;
  auto launch_forward = [&]() {
    return p->monitoring ? launch_gemm_dtype<false, true, EPI_FWD, true>(p->dtype, ta, tb, tc, gp, sms, st, pair)
                         : launch_gemm_dtype<false, true, EPI_FWD, false>(p->dtype, ta, tb, tc, gp, sms, st, pair);
  };
  auto run_forward = [&]() {  // timed when profiling is on; the conditional re-run below is not
    ProfScope prof(PROF_FWD, st);
    return launch_forward();
  };

  if (!row_reference_mode(p)) {
    if ((v = run_forward()) != LCE_OK) return v;
    if (p->monitoring)
      row_stats_kernel<true><<<blocks, 256, 0, st>>>(gp.tile_max, gp.tile_sum, gp.tile_ez, gp.tile_sq,
                                                     gp.target_logit, lab, (int)rows, gp.n_tiles, p->chunk_rows,
                                                     p->ignore_index, p->vocab_offset, p->vocab_local, parts);
    else
      row_stats_kernel<false><<<blocks, 256, 0, st>>>(gp.tile_max, gp.tile_sum, gp.tile_ez, gp.tile_sq,
                                                      gp.target_logit, lab, (int)rows, gp.n_tiles, p->chunk_rows,
                                                      p->ignore_index, p->vocab_offset, p->vocab_local, parts);
    return check_launch();
  }

  // Row-reference mode. A probe -- the forward kernel over the first two vocabulary tiles only, statistics
  // without slab -- gives each row a reference near its maximum (probe_ref_kernel). Then the forward proper;
  // then, only if some row's max logit turns out to lie outside the window around its reference (the
  // statistics kernel reports it through the device flag `rescue`), the same two kernels again with
  // reference = row max. That second pair returns at once when the flag is clear.
  int* rescue = w.rescue_flag;
  // Small vocabularies (below 64 tiles = 16384 columns) skip the probe: reference 0, and the conditional re-run --
  // cheap at that size -- covers rows whose logits lie outside the window; two launches fewer per chunk.
  const bool probe = gp.n_tiles >= 64;
  if (probe) {
    GemmParams pp = gp;
    pp.n_tiles = kProbeTiles;
    pp.store_slab = 0;
    if ((v = launch_gemm_dtype<false, true, EPI_FWD, false>(p->dtype, ta, tb, tc, pp, sms, st, pair)) != LCE_OK) return v;
    probe_ref_kernel<<<(int)((rows + 255) / 256), 256, 0, st>>>(gp.tile_max, p->chunk_rows, kProbeTiles, (int)rows,
                                                               w.row_ref + local0);
    if ((v = check_launch()) != LCE_OK) return v;
  }
  for (int pass = 0; pass < 2; ++pass) {
    const int* run_if = pass == 0 ? nullptr : rescue;
    const float* ref_in = (pass == 0 && !probe) ? nullptr : w.row_ref + local0;
    gp.row_ref = ref_in;
    gp.run_if = run_if;
    gp.run_mask = pass == 0 ? nullptr : w.rescue_groups;  // the re-run only touches the flagged 256-row groups
    gp.run_mask_row0 = (int)local0;
    if ((v = (pass == 0 ? run_forward() : launch_forward())) != LCE_OK) return v;
    if (p->monitoring)
      row_stats_rowref_kernel<true><<<blocks, 256, 0, st>>>(
          gp.tile_max, gp.tile_sum, gp.tile_ez, gp.tile_sq, gp.target_logit, lab, (int)rows, gp.n_tiles,
          p->chunk_rows, p->ignore_index, p->vocab_offset, p->vocab_local, ref_in, w.row_ref + local0,
          w.row_base + local0, rescue, w.rescue_groups, (int)local0, run_if, parts);
    else
      row_stats_rowref_kernel<false><<<blocks, 256, 0, st>>>(
          gp.tile_max, gp.tile_sum, gp.tile_ez, gp.tile_sq, gp.target_logit, lab, (int)rows, gp.n_tiles,
          p->chunk_rows, p->ignore_index, p->vocab_offset, p->vocab_local, ref_in, w.row_ref + local0,
          w.row_base + local0, rescue, w.rescue_groups, (int)local0, run_if, parts);
    if ((v = check_launch()) != LCE_OK) return v;
  }
  return LCE_OK;
}

int lce_combine_chunk(const lce_problem* p, const float* row_parts_all, const int64_t* labels, int64_t row0,
                      int64_t rows, void* workspace, void* stream) {
  int v = validate_problem(p);
  if (v != LCE_OK) return v;
  if ((v = check_chunk(p, row0, rows)) != LCE_OK) return v;
  if (!row_parts_all || !labels || !workspace) return LCE_ERR_INVALID_ARGUMENT;
  int sms = 0;
  if ((v = ensure_device(&sms)) != LCE_OK) return v;
  const Workspace w = layout_workspace(p, workspace, sms, chunk_buffer_of(p, row0));
  const long long local0 = row0 % p->chunk_rows;
  combine_kernel<<<1, 1024, 0, (cudaStream_t)stream>>>(row_parts_all + local0, p->world,
                                                       reinterpret_cast<const long long*>(labels) + row0, (int)rows,
                                                       p->chunk_rows, p->ignore_index, p->monitoring, w.lse + local0,
                                                       w.scalars, w.rescue_groups, w.n_rescue);
  return check_launch();
}

int lce_parts_bytes(const lce_problem* p, size_t* bytes) {
  const int v = validate_problem(p);
  if (v != LCE_OK) return v;
  if (!bytes || p->world > kMaxPeers) return LCE_ERR_INVALID_ARGUMENT;
  *bytes = kPeerFlagBytes + (size_t)kPartsSlots * parts_slot_bytes(p->world, p->chunk_rows);
  return LCE_OK;
}

static int check_parts_peers(const lce_problem* p, const lce_peer_table* peers) {
  if (!peers) return LCE_ERR_INVALID_ARGUMENT;
  if (peers->world != p->world || peers->world < 1 || peers->world > kMaxPeers) return LCE_ERR_INVALID_ARGUMENT;
  if (peers->rank < 0 || peers->rank >= peers->world) return LCE_ERR_INVALID_ARGUMENT;
  for (int g = 0; g < peers->world; ++g) {
    if (!peers->base[g]) return LCE_ERR_INVALID_ARGUMENT;
    if ((reinterpret_cast<uintptr_t>(peers->base[g]) & 255u) != 0) return LCE_ERR_MISALIGNED;
  }
  return LCE_OK;
}

int lce_parts_push(const lce_problem* p, const float* row_parts_local, int64_t row0, int64_t rows,
                   const lce_peer_table* peers, uint32_t epoch, void* stream) {
  int v = validate_problem(p);
  if (v != LCE_OK) return v;
  if ((v = check_chunk(p, row0, rows)) != LCE_OK) return v;
  if (!row_parts_local) return LCE_ERR_INVALID_ARGUMENT;
  if ((v = check_parts_peers(p, peers)) != LCE_OK) return v;
  cudaStream_t st = (cudaStream_t)stream;
  PeerBases bases;
  for (int g = 0; g < kMaxPeers; ++g)
    bases.base[g] = g < peers->world ? reinterpret_cast<unsigned char*>(peers->base[g]) : nullptr;
  const long long total = (long long)ROW_PARTS * rows * peers->world;
  const int grid = grid_for(total, 256, sm_count_or_default(), 1);
  parts_push_kernel<<<grid, 256, 0, st>>>(bases, peers->world, peers->rank, row_parts_local, p->chunk_rows,
                                          (int)(row0 % p->chunk_rows), (int)rows,
                                          parts_slot_off(p->world, p->chunk_rows, epoch));
  if ((v = check_launch()) != LCE_OK) return v;
  peer_signal_kernel<<<1, 32, 0, st>>>(bases, peers->world, peers->rank, 0, epoch, nullptr);
  return check_launch();
}

int lce_combine_chunk_peer(const lce_problem* p, const lce_peer_table* peers, uint32_t epoch, const int64_t* labels,
                           int64_t row0, int64_t rows, void* workspace, int32_t wait_ms, void* stream) {
  int v = validate_problem(p);
  if (v != LCE_OK) return v;
  if ((v = check_chunk(p, row0, rows)) != LCE_OK) return v;
  if (!labels || !workspace) return LCE_ERR_INVALID_ARGUMENT;
  if ((v = check_parts_peers(p, peers)) != LCE_OK) return v;
  int sms = 0;
  if ((v = ensure_device(&sms)) != LCE_OK) return v;
  const Workspace w = layout_workspace(p, workspace, sms, chunk_buffer_of(p, row0));
  const long long local0 = row0 % p->chunk_rows;
  const unsigned char* mine = reinterpret_cast<const unsigned char*>(peers->base[peers->rank]);
  const float* parts_all = reinterpret_cast<const float*>(mine + parts_slot_off(p->world, p->chunk_rows, epoch));
  const long long limit = (long long)(wait_ms > 0 ? wait_ms : 10000) * 1000000LL;
  combine_peer_kernel<<<1, 1024, 0, (cudaStream_t)stream>>>(
      reinterpret_cast<const uint32_t*>(mine), epoch, limit, parts_all + local0, p->world,
      reinterpret_cast<const long long*>(labels) + row0, (int)rows, p->chunk_rows, p->ignore_index, p->monitoring,
      w.lse + local0, w.scalars, w.rescue_groups, w.n_rescue);
  return check_launch();
}

int lce_dz_chunk(const lce_problem* p, const void* x, int64_t x_ld, const int64_t* labels, int64_t row0,
                 int64_t rows, void* workspace, void* stream) {
  int v = validate_problem(p);
  if (v != LCE_OK) return v;
  if ((v = check_chunk(p, row0, rows)) != LCE_OK) return v;
  if (!p->want_grad || !x || !labels || !workspace || x_ld < p->hidden) return LCE_ERR_INVALID_ARGUMENT;
  int sms = 0;
  if ((v = ensure_device(&sms)) != LCE_OK) return v;
  cudaStream_t st = (cudaStream_t)stream;
  const Workspace w = layout_workspace(p, workspace, sms, chunk_buffer_of(p, row0));
  const int es = elem_size(p->dtype);
  const long long v_pad = vocab_pad(p), h_pad = hidden_pad(p);
  const long long rows_pad = round_up(rows, BLOCK_M);
  const int n_vtiles = (int)(v_pad / BLOCK_N);
  const long long local0 = row0 % p->chunk_rows;
  const long long* lab = reinterpret_cast<const long long*>(labels) + row0;
  char* slab = reinterpret_cast<char*>(w.slab) + (size_t)local0 * (size_t)v_pad * es;
  if (row_reference_mode(p)) {
    // per-row factor, scaled copy of the x rows, label entry of the slab: see row_finish_kernel
    const char* xrows = reinterpret_cast<const char*>(x) + (size_t)row0 * (size_t)x_ld * es;
    char* xs = reinterpret_cast<char*>(w.xs) + (size_t)local0 * (size_t)h_pad * es;
    if (p->dtype == LCE_DTYPE_BF16)
      row_finish_kernel<__nv_bfloat16><<<(int)rows_pad, 256, 0, st>>>(
          reinterpret_cast<const __nv_bfloat16*>(xrows), x_ld, reinterpret_cast<__nv_bfloat16*>(xs), h_pad,
          (int)p->hidden, reinterpret_cast<__nv_bfloat16*>(slab), v_pad, w.row_base + local0, w.lse + local0, lab,
          (int)rows, p->ignore_index, p->vocab_offset, p->vocab_local, p->z_regularization, w.row_coef + local0);
    else
      row_finish_kernel<float><<<(int)rows_pad, 256, 0, st>>>(
          reinterpret_cast<const float*>(xrows), x_ld, reinterpret_cast<float*>(xs), h_pad, (int)p->hidden,
          reinterpret_cast<float*>(slab), v_pad, w.row_base + local0, w.lse + local0, lab, (int)rows,
          p->ignore_index, p->vocab_offset, p->vocab_local, p->z_regularization, w.row_coef + local0);
    return check_launch();
  }
  const long long items = (rows_pad / 8) * n_vtiles;
  const int grid = grid_for(items, 1, sms, 16);
  switch (p->dtype) {
    case LCE_DTYPE_F16:
      dz_transform_kernel<__half><<<grid, 256, 0, st>>>(reinterpret_cast<__half*>(slab), v_pad, w.tile_max + local0,
                                                        w.lse + local0, lab, (int)rows_pad, (int)rows, n_vtiles,
                                                        p->chunk_rows, p->ignore_index, p->vocab_offset,
                                                        p->z_regularization);
      break;
    case LCE_DTYPE_BF16:
      dz_transform_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(
          reinterpret_cast<__nv_bfloat16*>(slab), v_pad, w.tile_max + local0, w.lse + local0, lab, (int)rows_pad,
          (int)rows, n_vtiles, p->chunk_rows, p->ignore_index, p->vocab_offset, p->z_regularization);
      break;
    default:
      dz_transform_kernel<float><<<grid, 256, 0, st>>>(reinterpret_cast<float*>(slab), v_pad, w.tile_max + local0,
                                                       w.lse + local0, lab, (int)rows_pad, (int)rows, n_vtiles,
                                                       p->chunk_rows, p->ignore_index, p->vocab_offset,
                                                       p->z_regularization);
  }
  return check_launch();
}

}  // extern "C"

namespace {

// Where the dx contraction sends its output tiles when the partials are exchanged between ranks.
struct PeerScatter {
  PeerBases bases;
  PeerLayout layout;
  int world, rank, buf;
};

PeerLayout layout_peer(const lce_problem* p, int dx_dtype, int splits) {
  PeerLayout l;
  l.slots = p->world * splits;
  l.rows_own = (int)(p->chunk_rows / p->world);
  l.recv_bytes = round_up((long long)l.slots * l.rows_own * hidden_pad(p) * (long long)sizeof(float), 1024);
  l.stage_bytes = round_up(p->chunk_rows * p->hidden * (long long)elem_size(dx_dtype), 1024);
  l.total = kPeerFlagBytes + 2 * l.recv_bytes + 2 * l.stage_bytes;
  return l;
}

int check_peers(const lce_problem* p, const lce_peer_table* peers, int dx_dtype) {
  if (!peers) return LCE_ERR_INVALID_ARGUMENT;
  if (dx_dtype != LCE_DTYPE_F16 && dx_dtype != LCE_DTYPE_BF16 && dx_dtype != LCE_DTYPE_F32)
    return LCE_ERR_INVALID_ARGUMENT;
  if (peers->world != p->world || peers->world < 1 || peers->world > kMaxPeers) return LCE_ERR_INVALID_ARGUMENT;
  if (peers->rank < 0 || peers->rank >= peers->world) return LCE_ERR_INVALID_ARGUMENT;
  if (p->chunk_rows % ((long long)BLOCK_M * peers->world) != 0) return LCE_ERR_UNSUPPORTED_SHAPE;
  for (int g = 0; g < peers->world; ++g) {
    if (!peers->base[g]) return LCE_ERR_INVALID_ARGUMENT;
    if ((reinterpret_cast<uintptr_t>(peers->base[g]) & 255u) != 0) return LCE_ERR_MISALIGNED;
  }
  return LCE_OK;
}

PeerBases bases_of(const lce_peer_table* peers) {
  PeerBases b;
  for (int g = 0; g < kMaxPeers; ++g)
    b.base[g] = g < peers->world ? reinterpret_cast<unsigned char*>(peers->base[g]) : nullptr;
  return b;
}

// partials[s] = dZ * W^T over K-split s of the vocabulary, scaled by logit_scale / n_valid: into the workspace
// (scatter == nullptr) or into the owners' receive buffers.
// direct_dx (optional, one split only): the rows of dx themselves, element type of x, row stride direct_ld; the
// epilogue then writes them instead of fp32 partials.
int launch_dx_gemm(const lce_problem* p, const void* weight, int64_t w_ld, int64_t row0, int64_t rows,
                   const Workspace& w, int sms, cudaStream_t st, const PeerScatter* scatter, void* direct_dx = nullptr,
                   int64_t direct_ld = 0) {
  const int es = elem_size(p->dtype);
  const long long local0 = row0 % p->chunk_rows;
  const long long v_pad = vocab_pad(p), h_pad = hidden_pad(p);
  const long long rows_pad = round_up(rows, BLOCK_M);
  const bool pair = use_pair_kernel(rows_pad / BLOCK_M, sms);
  CUtensorMap ta, tb;
  int v;
  if ((v = make_operand_tmap(&ta, p->dtype, false, w.slab, v_pad, p->chunk_rows, v_pad, BLOCK_M)) != LCE_OK) return v;
  if ((v = make_operand_tmap(&tb, p->dtype, false, weight, p->vocab_local, p->hidden, w_ld, rows_of_b_tile(pair))) !=
      LCE_OK)
    return v;
  GemmParams gp;
  memset(&gp, 0, sizeof(gp));
  gp.m_tiles = (int)(rows_pad / BLOCK_M);
  gp.n_tiles = (int)(h_pad / BLOCK_N);
  gp.splits = w.dx_splits;
  gp.k_blocks = (int)(v_pad * es / 128 / w.dx_splits);
  gp.a_mn0 = (int)local0;
  // N-first: the units in flight at one time then cover all H tiles of a few row blocks, so each slab row block is
  // streamed from DRAM once and only the (smaller) weight is re-read per group of row blocks
  gp.n_fastest = 1;
  gp.out = w.dx_part + local0 * h_pad;  // padded partial buffer: whole tiles are stored, the reduction reads what exists
  gp.out_ld = h_pad;
  gp.out_split_stride = (long long)p->chunk_rows * h_pad;
  gp.out_rows = (int)rows_pad;
  gp.out_cols = (int)h_pad;
  gp.out_vector_ok = 1;
  gp.accumulate = 0;
  gp.out_scale = p->logit_scale;
  gp.out_div = &w.scalars->n_valid;
  gp.row_coef = row_reference_mode(p) ? w.row_coef + local0 : nullptr;
  gp.status = &w.scalars->status;
  CUtensorMap tc = ta;
  if (direct_dx != nullptr) {
    // plain conversion and store of coef * row_coef * acc; rows and columns beyond dx are masked
    char* rows0 = reinterpret_cast<char*>(direct_dx) + (size_t)row0 * (size_t)direct_ld * es;
    gp.out_sum = rows0;
    gp.out_res = nullptr;
    gp.out_pair_ld = direct_ld;
    gp.out_pair_last = 1;
    gp.out_rows = (int)rows;
    gp.out_cols = (int)p->hidden;
    gp.out_vector_ok = ((reinterpret_cast<uintptr_t>(rows0) & 31u) == 0 && ((direct_ld * es) & 31) == 0) ? 1 : 0;
  } else if (scatter == nullptr && epilogue_tma_enabled()) {
    // the partials [splits][chunk_rows][h_pad] seen as one fp32 matrix of splits * chunk_rows rows
    if ((v = make_store_tmap(&tc, LCE_DTYPE_F32, w.dx_part, h_pad, (long long)w.dx_splits * p->chunk_rows, h_pad)) !=
        LCE_OK)
      return v;
    gp.out_tma = 1;
    gp.c_row0 = (int)local0;
    gp.c_split_rows = (int)p->chunk_rows;
  }
  if (scatter != nullptr) {
    for (int g = 0; g < scatter->world; ++g)
      gp.peer_out[g] = reinterpret_cast<float*>(scatter->bases.base[g] + scatter->layout.recv_off(scatter->buf));
    gp.peer_rows_own = scatter->layout.rows_own;
    gp.peer_row0 = (int)local0;
    gp.peer_slot0 = scatter->rank * w.dx_splits;
  }
  ProfScope prof(PROF_DX, st);
  return launch_gemm_dtype<false, false, EPI_F32, false>(p->dtype, ta, tb, tc, gp, sms, st, pair);
}

long long peer_wait_limit_ns(int32_t wait_ms) { return (long long)(wait_ms > 0 ? wait_ms : 10000) * 1000000LL; }

}  // namespace

extern "C" {

int lce_dx_chunk(const lce_problem* p, const void* weight, int64_t w_ld, int64_t row0, int64_t rows, void* workspace,
                 void* dx, int64_t dx_ld, int32_t dx_dtype, void* stream) {
  int v = validate_problem(p);
  if (v != LCE_OK) return v;
  if ((v = check_chunk(p, row0, rows)) != LCE_OK) return v;
  if (!p->want_grad || !weight || !workspace || !dx) return LCE_ERR_INVALID_ARGUMENT;
  if (w_ld < p->vocab_local || dx_ld < p->hidden) return LCE_ERR_INVALID_ARGUMENT;
  if (dx_dtype != LCE_DTYPE_F16 && dx_dtype != LCE_DTYPE_BF16 && dx_dtype != LCE_DTYPE_F32)
    return LCE_ERR_INVALID_ARGUMENT;
  int sms = 0;
  if ((v = ensure_device(&sms)) != LCE_OK) return v;
  cudaStream_t st = (cudaStream_t)stream;
  const Workspace w = layout_workspace(p, workspace, sms, chunk_buffer_of(p, row0));
  const long long local0 = row0 % p->chunk_rows;
  const long long h_pad = hidden_pad(p);
  if (w.dx_splits == 1 && dx_dtype == p->dtype) {
    // one split: the contraction's epilogue scales, converts and stores the dx rows itself
    return launch_dx_gemm(p, weight, w_ld, row0, rows, w, sms, st, nullptr, dx, dx_ld);
  }
  if ((v = launch_dx_gemm(p, weight, w_ld, row0, rows, w, sms, st, nullptr)) != LCE_OK) return v;

  // fixed-order sum of the partials -> dx rows
  const float* part = w.dx_part + local0 * h_pad;
  const long long quads = rows * (p->hidden / 4);
  const int grid = grid_for(quads, 256, sms, 8);
  const long long ss = (long long)p->chunk_rows * h_pad;
  char* dx_rows = reinterpret_cast<char*>(dx) + (size_t)row0 * (size_t)dx_ld * elem_size(dx_dtype);
  switch (dx_dtype) {
    case LCE_DTYPE_F16:
      dx_reduce_kernel<__half><<<grid, 256, 0, st>>>(part, w.dx_splits, ss, h_pad, (int)rows, (int)p->hidden,
                                                     reinterpret_cast<__half*>(dx_rows), dx_ld);
      break;
    case LCE_DTYPE_BF16:
      dx_reduce_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(part, w.dx_splits, ss, h_pad, (int)rows, (int)p->hidden,
                                                            reinterpret_cast<__nv_bfloat16*>(dx_rows), dx_ld);
      break;
    default:
      dx_reduce_kernel<float><<<grid, 256, 0, st>>>(part, w.dx_splits, ss, h_pad, (int)rows, (int)p->hidden,
                                                    reinterpret_cast<float*>(dx_rows), dx_ld);
  }
  return check_launch();
}

int lce_peer_bytes(const lce_problem* p, int32_t dx_dtype, size_t* bytes) {
  int v = validate_problem(p);
  if (v != LCE_OK) return v;
  if (!bytes) return LCE_ERR_INVALID_ARGUMENT;
  if (dx_dtype != LCE_DTYPE_F16 && dx_dtype != LCE_DTYPE_BF16 && dx_dtype != LCE_DTYPE_F32)
    return LCE_ERR_INVALID_ARGUMENT;
  if (p->world < 1 || p->world > kMaxPeers) return LCE_ERR_INVALID_ARGUMENT;
  if (p->chunk_rows % ((long long)BLOCK_M * p->world) != 0) return LCE_ERR_UNSUPPORTED_SHAPE;
  int sms = 0;
  if ((v = ensure_device(&sms)) != LCE_OK) return v;
  *bytes = layout_peer(p, dx_dtype, choose_dx_splits(p, sms)).total;
  return LCE_OK;
}

int lce_dx_chunk_peer(const lce_problem* p, const void* weight, int64_t w_ld, int64_t row0, int64_t rows,
                      void* workspace, const lce_peer_table* peers, int32_t dx_dtype, uint32_t epoch, void* stream) {
  int v = validate_problem(p);
  if (v != LCE_OK) return v;
  if ((v = check_chunk(p, row0, rows)) != LCE_OK) return v;
  if (!p->want_grad || !weight || !workspace) return LCE_ERR_INVALID_ARGUMENT;
  if (w_ld < p->vocab_local) return LCE_ERR_INVALID_ARGUMENT;
  if ((v = check_peers(p, peers, dx_dtype)) != LCE_OK) return v;
  int sms = 0;
  if ((v = ensure_device(&sms)) != LCE_OK) return v;
  cudaStream_t st = (cudaStream_t)stream;
  const Workspace w = layout_workspace(p, workspace, sms, chunk_buffer_of(p, row0));
  PeerScatter sc;
  sc.bases = bases_of(peers);
  sc.layout = layout_peer(p, dx_dtype, w.dx_splits);
  sc.world = peers->world;
  sc.rank = peers->rank;
  sc.buf = (int)(epoch & 1u);
  if ((v = launch_dx_gemm(p, weight, w_ld, row0, rows, w, sms, st, &sc)) != LCE_OK) return v;
  peer_signal_kernel<<<1, 32, 0, st>>>(sc.bases, sc.world, sc.rank, 0, epoch, nullptr);
  return check_launch();
}

int lce_dx_reduce_peer(const lce_problem* p, int64_t row0, int64_t rows, void* workspace, const lce_peer_table* peers,
                       int32_t dx_dtype, uint32_t epoch, int32_t wait_ms, void* stream) {
  int v = validate_problem(p);
  if (v != LCE_OK) return v;
  if ((v = check_chunk(p, row0, rows)) != LCE_OK) return v;
  if (!p->want_grad || !workspace) return LCE_ERR_INVALID_ARGUMENT;
  if ((v = check_peers(p, peers, dx_dtype)) != LCE_OK) return v;
  int sms = 0;
  if ((v = ensure_device(&sms)) != LCE_OK) return v;
  cudaStream_t st = (cudaStream_t)stream;
  const Workspace w = layout_workspace(p, workspace, sms, chunk_buffer_of(p, row0));
  const PeerBases bases = bases_of(peers);
  const PeerLayout l = layout_peer(p, dx_dtype, w.dx_splits);
  const int buf = (int)(epoch & 1u);
  const int rank = peers->rank;
  // rows of this launch that this rank owns, as indices into its owned slice
  const long long local0 = row0 % p->chunk_rows;
  const long long lo = std::max<long long>(local0, (long long)rank * l.rows_own);
  const long long hi = std::min<long long>(local0 + rows, (long long)(rank + 1) * l.rows_own);
  const int own_lo = (int)(lo - (long long)rank * l.rows_own);
  const int own_hi = hi > lo ? (int)(hi - (long long)rank * l.rows_own) : own_lo;
  unsigned char* mine = bases.base[rank];
  const uint32_t* flags_a = reinterpret_cast<const uint32_t*>(mine);
  const float* recv = reinterpret_cast<const float*>(mine + l.recv_off(buf));
  const long long octs = (long long)(own_hi - own_lo) * (p->hidden / 8);
  const int grid = grid_for(octs > 0 ? octs : 1, 256, sms, 4);
  const long long limit = peer_wait_limit_ns(wait_ms);
  const int ld = (int)hidden_pad(p);
  switch (dx_dtype) {
    case LCE_DTYPE_F16:
      peer_reduce_push_kernel<__half><<<grid, 256, 0, st>>>(bases, peers->world, flags_a, epoch, limit, recv, l.slots,
                                                            l.rows_own, ld, own_lo, own_hi, rank * l.rows_own,
                                                            (int)p->hidden, l.stage_off(buf), &w.scalars->status);
      break;
    case LCE_DTYPE_BF16:
      peer_reduce_push_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(bases, peers->world, flags_a, epoch, limit, recv,
                                                                   l.slots, l.rows_own, ld, own_lo, own_hi,
                                                                   rank * l.rows_own, (int)p->hidden, l.stage_off(buf),
                                                                   &w.scalars->status);
      break;
    default:
      peer_reduce_push_kernel<float><<<grid, 256, 0, st>>>(bases, peers->world, flags_a, epoch, limit, recv, l.slots,
                                                           l.rows_own, ld, own_lo, own_hi, rank * l.rows_own,
                                                           (int)p->hidden, l.stage_off(buf), &w.scalars->status);
  }
  if ((v = check_launch()) != LCE_OK) return v;
  // not published when the wait above ran out (status word set): nothing was staged, so nobody may copy
  peer_signal_kernel<<<1, 32, 0, st>>>(bases, peers->world, rank, 1, epoch, &w.scalars->status);
  return check_launch();
}

int lce_dx_finish_peer(const lce_problem* p, int64_t row0, int64_t rows, void* workspace, const lce_peer_table* peers,
                       uint32_t epoch, void* dx, int64_t dx_ld, int32_t dx_dtype, int32_t wait_ms, void* stream) {
  int v = validate_problem(p);
  if (v != LCE_OK) return v;
  if ((v = check_chunk(p, row0, rows)) != LCE_OK) return v;
  if (!p->want_grad || !workspace || !dx || dx_ld < p->hidden) return LCE_ERR_INVALID_ARGUMENT;
  if ((v = check_peers(p, peers, dx_dtype)) != LCE_OK) return v;
  const int des = elem_size(dx_dtype);
  if ((reinterpret_cast<uintptr_t>(dx) & 15u) != 0 || ((dx_ld * des) & 15) != 0) return LCE_ERR_MISALIGNED;
  int sms = 0;
  if ((v = ensure_device(&sms)) != LCE_OK) return v;
  cudaStream_t st = (cudaStream_t)stream;
  const Workspace w = layout_workspace(p, workspace, sms, chunk_buffer_of(p, row0));
  const PeerLayout l = layout_peer(p, dx_dtype, w.dx_splits);
  const int buf = (int)(epoch & 1u);
  unsigned char* mine = reinterpret_cast<unsigned char*>(peers->base[peers->rank]);
  const uint32_t* flags_b = reinterpret_cast<const uint32_t*>(mine) + kMaxPeers;
  const long long local0 = row0 % p->chunk_rows;
  const long long octs = rows * (p->hidden / 8);
  const int grid = grid_for(octs, 256, sms, 4);
  const long long limit = peer_wait_limit_ns(wait_ms);
  char* dx_rows = reinterpret_cast<char*>(dx) + (size_t)row0 * (size_t)dx_ld * des;
  const unsigned char* stage = mine + l.stage_off(buf);
  switch (dx_dtype) {
    case LCE_DTYPE_F16:
      peer_finish_kernel<__half><<<grid, 256, 0, st>>>(flags_b, peers->world, epoch, limit,
                                                       reinterpret_cast<const __half*>(stage), (int)local0, (int)rows,
                                                       (int)p->hidden, reinterpret_cast<__half*>(dx_rows), dx_ld,
                                                       &w.scalars->status);
      break;
    case LCE_DTYPE_BF16:
      peer_finish_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(
          flags_b, peers->world, epoch, limit, reinterpret_cast<const __nv_bfloat16*>(stage), (int)local0, (int)rows,
          (int)p->hidden, reinterpret_cast<__nv_bfloat16*>(dx_rows), dx_ld, &w.scalars->status);
      break;
    default:
      peer_finish_kernel<float><<<grid, 256, 0, st>>>(flags_b, peers->world, epoch, limit,
                                                      reinterpret_cast<const float*>(stage), (int)local0, (int)rows,
                                                      (int)p->hidden, reinterpret_cast<float*>(dx_rows), dx_ld,
                                                      &w.scalars->status);
  }
  return check_launch();
}

int lce_dw_chunk(const lce_problem* p, const void* x, int64_t x_ld, int64_t row0, int64_t rows, void* workspace,
                 void* dweight, int64_t dw_ld, void* dweight_residual, int64_t dwr_ld, int32_t first, int32_t last,
                 void* stream) {
  int v = validate_problem(p);
  if (v != LCE_OK) return v;
  if ((v = check_chunk(p, row0, rows)) != LCE_OK) return v;
  if (!p->want_grad || !x || !workspace || !dweight) return LCE_ERR_INVALID_ARGUMENT;
  if (x_ld < p->hidden || dw_ld < p->vocab_local) return LCE_ERR_INVALID_ARGUMENT;
  const int es = elem_size(p->dtype);
  // 16-bit types carry the sum over the chunks as dweight + dweight_residual; a pass of one call needs no residual,
  // and an fp32 dweight is its own accumulator
  const bool sum_pair = p->dtype != LCE_DTYPE_F32;
  const bool need_res = sum_pair && !(first && last);
  if (need_res && (!dweight_residual || dwr_ld != dw_ld)) return LCE_ERR_INVALID_ARGUMENT;
  if ((reinterpret_cast<uintptr_t>(dweight) & (uintptr_t)(es - 1)) != 0 ||
      (need_res && (reinterpret_cast<uintptr_t>(dweight_residual) & (uintptr_t)(es - 1)) != 0))
    return LCE_ERR_MISALIGNED;
  int sms = 0;
  if ((v = ensure_device(&sms)) != LCE_OK) return v;
  cudaStream_t st = (cudaStream_t)stream;
  const Workspace w = layout_workspace(p, workspace, sms, chunk_buffer_of(p, row0));
  const long long local0 = row0 % p->chunk_rows;

  // dW (+)= x^T * dZ, scaled by logit_scale / n_valid
  const long long v_pad = vocab_pad(p), h_pad = hidden_pad(p);
  const long long rows_pad = round_up(rows, BLOCK_M);
  const bool pair = use_pair_kernel(h_pad / BLOCK_M, sms);
  const bool rowref = row_reference_mode(p);
  CUtensorMap ta, tb;
  // A operand (M = hidden, K = rows): the x rows themselves, or in row-reference mode their scaled copy. Both maps
  // describe only what exists; TMA returns zeros for hidden columns / rows beyond it.
  v = rowref ? make_operand_tmap(&ta, p->dtype, true, w.xs, p->hidden, p->chunk_rows, h_pad, BLOCK_M)
             : make_operand_tmap(&ta, p->dtype, true, x, p->hidden, p->n_rows_total, x_ld, BLOCK_M);
  if (v != LCE_OK) return v;
  if ((v = make_operand_tmap(&tb, p->dtype, true, w.slab, v_pad, p->chunk_rows, v_pad, rows_of_b_tile(pair))) != LCE_OK)
    return v;
  // 32-byte epilogue accesses need 32-byte aligned rows in the outputs; otherwise the epilogue goes element-wise
  auto rows_aligned32 = [](const void* ptr, long long ld_bytes) {
    return ptr == nullptr || ((reinterpret_cast<uintptr_t>(ptr) & 31u) == 0 && (ld_bytes & 31) == 0);
  };
  GemmParams gp;
  memset(&gp, 0, sizeof(gp));
  gp.m_tiles = (int)(h_pad / BLOCK_M);
  gp.n_tiles = (int)(v_pad / BLOCK_N);
  gp.splits = 1;
  gp.k_blocks = (int)(rows_pad * es / 128);
  gp.out_rows = (int)p->hidden;
  gp.out_cols = (int)p->vocab_local;
  gp.out_vector_ok =
      (rows_aligned32(dweight, dw_ld * es) && rows_aligned32(need_res ? dweight_residual : nullptr, dw_ld * es)) ? 1 : 0;
  gp.a_k0 = (int)(rowref ? local0 : row0);
  gp.b_k0 = (int)local0;
  gp.accumulate = first ? 0 : 1;
  gp.out_scale = p->logit_scale;
  gp.out_div = &w.scalars->n_valid;
  gp.status = &w.scalars->status;
  CUtensorMap tc = ta;
  if (sum_pair) {
    gp.out_sum = dweight;
    gp.out_res = need_res ? dweight_residual : nullptr;
    gp.out_pair_ld = dw_ld;
    gp.out_pair_last = last ? 1 : 0;
  } else {
    gp.out = reinterpret_cast<float*>(dweight);
    gp.out_ld = dw_ld;
    // A chunk that only writes the fp32 result does it through shared memory and TMA tile stores. Chunks that add
    // to it read-add-store in the epilogue: TMA reduce-adds (performed at the memory side) were measured 3 % slower
    // for this kernel (1264 against 1300 TFLOP/s at 4096 x 2048 x 131072).
    if (first && epilogue_tma_enabled() && (reinterpret_cast<uintptr_t>(dweight) & 15u) == 0 &&
        ((dw_ld * 4) & 15) == 0) {
      if ((v = make_store_tmap(&tc, LCE_DTYPE_F32, dweight, p->vocab_local, p->hidden, dw_ld)) != LCE_OK) return v;
      gp.out_tma = 1;
    }
  }
  {
    ProfScope prof(PROF_DW, st);
    v = launch_gemm_dtype<true, true, EPI_F32, false>(p->dtype, ta, tb, tc, gp, sms, st, pair);
  }
  return v;
}

int lce_backward_chunk(const lce_problem* p, const void* x, int64_t x_ld, const void* weight, int64_t w_ld,
                       const int64_t* labels, int64_t row0, int64_t rows, void* workspace, void* dx, int64_t dx_ld,
                       int32_t dx_dtype, void* dweight, int64_t dw_ld, void* dweight_residual, int64_t dwr_ld,
                       int32_t first, int32_t last, void* stream) {
  int v = lce_dz_chunk(p, x, x_ld, labels, row0, rows, workspace, stream);
  if (v != LCE_OK) return v;
  if ((v = lce_dx_chunk(p, weight, w_ld, row0, rows, workspace, dx, dx_ld, dx_dtype, stream)) != LCE_OK) return v;
  return lce_dw_chunk(p, x, x_ld, row0, rows, workspace, dweight, dw_ld, dweight_residual, dwr_ld, first, last,
                      stream);
}

int lce_fused_pass(const lce_problem* p, const void* x, int64_t x_ld, const void* weight, int64_t w_ld,
                   const int64_t* labels, void* workspace, float* row_parts, void* dx, int64_t dx_ld, int32_t dx_dtype,
                   void* dweight, int64_t dw_ld, void* dweight_residual, int64_t dwr_ld, float* out5, void* stream) {
  int v = validate_problem(p);
  if (v != LCE_OK) return v;
  if (p->world != 1 || p->vocab_offset != 0) return LCE_ERR_INVALID_ARGUMENT;  // sharded callers exchange between the steps
  if (!x || !weight || !labels || !workspace || !row_parts || !out5) return LCE_ERR_INVALID_ARGUMENT;
  if (!p->want_grad && (dx || dweight)) return LCE_ERR_INVALID_ARGUMENT;
  if (p->want_grad && !dx && !dweight) return LCE_ERR_INVALID_ARGUMENT;
  if ((v = lce_begin(p, labels, workspace, stream)) != LCE_OK) return v;
  const int64_t n_chunks = (p->n_rows_total + p->chunk_rows - 1) / p->chunk_rows;
  for (int64_t ci = 0; ci < n_chunks; ++ci) {
    const int64_t row0 = ci * p->chunk_rows;
    const int64_t rows = std::min<int64_t>(p->chunk_rows, p->n_rows_total - row0);
    if ((v = lce_forward_chunk(p, x, x_ld, weight, w_ld, labels, row0, rows, workspace, row_parts, stream)) != LCE_OK)
      return v;
    if ((v = lce_combine_chunk(p, row_parts, labels, row0, rows, workspace, stream)) != LCE_OK) return v;
    if (!p->want_grad) continue;
    if ((v = lce_dz_chunk(p, x, x_ld, labels, row0, rows, workspace, stream)) != LCE_OK) return v;
    if (dx && (v = lce_dx_chunk(p, weight, w_ld, row0, rows, workspace, dx, dx_ld, dx_dtype, stream)) != LCE_OK) return v;
    if (dweight && (v = lce_dw_chunk(p, x, x_ld, row0, rows, workspace, dweight, dw_ld, dweight_residual, dwr_ld,
                                     ci == 0, ci == n_chunks - 1, stream)) != LCE_OK)
      return v;
  }
  return lce_finalize(p, workspace, out5, stream);
}

int lce_finalize(const lce_problem* p, void* workspace, float* out5, void* stream) {
  int v = validate_problem(p);
  if (v != LCE_OK) return v;
  if (!workspace || !out5) return LCE_ERR_INVALID_ARGUMENT;
  int sms = 0;
  if ((v = ensure_device(&sms)) != LCE_OK) return v;
  const Workspace w = layout_workspace(p, workspace, sms);
  finalize_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(w.scalars, (double)p->n_rows_total, p->z_regularization, out5);
  return check_launch();
}

}  // extern "C"

namespace {
template <typename S>
int scale_cast_dst(const S* src, long long src_ld, void* dst, int dst_dtype, long long dst_ld, long long rows,
                   long long cols, const float* f, int grid, cudaStream_t st, int skip) {
  switch (dst_dtype) {
    case LCE_DTYPE_F16:
      scale_cast_kernel<S, __half><<<grid, 256, 0, st>>>(src, src_ld, reinterpret_cast<__half*>(dst), dst_ld, rows,
                                                         cols, f, skip);
      break;
    case LCE_DTYPE_BF16:
      scale_cast_kernel<S, __nv_bfloat16><<<grid, 256, 0, st>>>(src, src_ld, reinterpret_cast<__nv_bfloat16*>(dst),
                                                                dst_ld, rows, cols, f, skip);
      break;
    case LCE_DTYPE_F32:
      scale_cast_kernel<S, float><<<grid, 256, 0, st>>>(src, src_ld, reinterpret_cast<float*>(dst), dst_ld, rows,
                                                        cols, f, skip);
      break;
    default: return LCE_ERR_INVALID_ARGUMENT;
  }
  return check_launch();
}
}  // namespace

extern "C" {

int lce_grad_scale_cast(const void* src, int32_t src_dtype, int64_t src_ld, void* dst, int32_t dst_dtype,
                        int64_t dst_ld, int64_t rows, int64_t cols, const float* dev_factor, void* stream) {
  if (!src || !dst || !dev_factor || rows <= 0 || cols <= 0 || src_ld < cols || dst_ld < cols)
    return LCE_ERR_INVALID_ARGUMENT;
  if (cols % 8 != 0) return LCE_ERR_UNSUPPORTED_SHAPE;
  auto aligned = [](const void* ptr, long long ld, int dtype) {
    const long long es = dtype == LCE_DTYPE_F32 ? 4 : 2;
    return (reinterpret_cast<uintptr_t>(ptr) & 15u) == 0 && ((ld * es) & 15) == 0;
  };
  if (!aligned(src, src_ld, src_dtype) || !aligned(dst, dst_ld, dst_dtype)) return LCE_ERR_MISALIGNED;
  const int sms = sm_count_or_default();
  const int grid = grid_for(rows * (cols / 8), 256, sms, 16);
  const int skip = (src == dst && src_dtype == dst_dtype) ? 1 : 0;
  cudaStream_t st = (cudaStream_t)stream;
  switch (src_dtype) {
    case LCE_DTYPE_F16:
      return scale_cast_dst(reinterpret_cast<const __half*>(src), src_ld, dst, dst_dtype, dst_ld, rows, cols,
                            dev_factor, grid, st, skip);
    case LCE_DTYPE_BF16:
      return scale_cast_dst(reinterpret_cast<const __nv_bfloat16*>(src), src_ld, dst, dst_dtype, dst_ld, rows, cols,
                            dev_factor, grid, st, skip);
    case LCE_DTYPE_F32:
      return scale_cast_dst(reinterpret_cast<const float*>(src), src_ld, dst, dst_dtype, dst_ld, rows, cols,
                            dev_factor, grid, st, skip);
  }
  return LCE_ERR_INVALID_ARGUMENT;
}

int lce_read_status(void* workspace, void* stream) {
  if (!workspace) return LCE_ERR_INVALID_ARGUMENT;
  PassScalars host;
  if (cudaMemcpyAsync(&host, workspace, sizeof(host), cudaMemcpyDeviceToHost, (cudaStream_t)stream) != cudaSuccess)
    return LCE_ERR_CUDA;
  if (cudaStreamSynchronize((cudaStream_t)stream) != cudaSuccess) return LCE_ERR_CUDA;
  return host.status == 0 ? LCE_OK : LCE_ERR_DEVICE_TIMEOUT;
}

int lce_rerun_stats_async(void* workspace, int32_t* host_out2, void* stream) {
  if (!workspace || !host_out2) return LCE_ERR_INVALID_ARGUMENT;
  const PassScalars* sc = reinterpret_cast<const PassScalars*>(workspace);
  static_assert(offsetof(PassScalars, seen_groups) == offsetof(PassScalars, rerun_groups) + sizeof(int), "pair");
  if (cudaMemcpyAsync(host_out2, &sc->rerun_groups, 2 * sizeof(int), cudaMemcpyDeviceToHost,
                      (cudaStream_t)stream) != cudaSuccess)
    return LCE_ERR_CUDA;
  return LCE_OK;
}

int lce_profile_enable(int32_t enable) {
  std::lock_guard<std::mutex> lock(g_prof_mutex);
  g_prof_enabled = enable != 0;
  return LCE_OK;
}

int lce_profile_read(double* ms3, long long* launches3) {
  if (!ms3 || !launches3) return LCE_ERR_INVALID_ARGUMENT;
  std::lock_guard<std::mutex> lock(g_prof_mutex);
  for (int k = 0; k < PROF_KINDS; ++k) {
    ms3[k] = 0.0;
    launches3[k] = 0;
  }
  int rc = LCE_OK;
  for (const ProfSpan& sp : g_prof_spans) {
    float ms = 0.f;
    if (cudaEventSynchronize(sp.stop) != cudaSuccess || cudaEventElapsedTime(&ms, sp.start, sp.stop) != cudaSuccess) {
      rc = LCE_ERR_CUDA;
    } else {
      ms3[sp.kind] += ms;
      launches3[sp.kind] += 1;
    }
    g_prof_free.push_back(sp);
  }
  g_prof_spans.clear();
  return rc;
}

int lce_debug_gemm(int32_t dtype, int32_t a_mn_major, int32_t b_mn_major, const void* a, int64_t a_ld, const void* b,
                   int64_t b_ld, float* out, int64_t m, int64_t n, int64_t k, int32_t splits, int32_t single_cta,
                   int32_t raster_group, int32_t n_fastest, int* dev_status, void* stream) {
  if (dtype != LCE_DTYPE_F16 && dtype != LCE_DTYPE_BF16 && dtype != LCE_DTYPE_F32) return LCE_ERR_INVALID_ARGUMENT;
  if (!a || !b || !out || !dev_status || m <= 0 || n <= 0 || k <= 0 || splits < 1) return LCE_ERR_INVALID_ARGUMENT;
  const int es = elem_size(dtype);
  const int bk = 128 / es;
  if (m % BLOCK_M != 0 || n % BLOCK_N != 0 || k % ((long long)bk * splits) != 0) return LCE_ERR_UNSUPPORTED_SHAPE;
  if (m > (1ll << 30) || n > (1ll << 30) || k > (1ll << 30)) return LCE_ERR_TOO_LARGE;
  int sms = 0;
  int v = ensure_device(&sms);
  if (v != LCE_OK) return v;
  const bool pair = !single_cta && use_pair_kernel(m / BLOCK_M, sms);
  CUtensorMap ta, tb;
  v = a_mn_major ? make_operand_tmap(&ta, dtype, true, a, m, k, a_ld, BLOCK_M)
                 : make_operand_tmap(&ta, dtype, false, a, k, m, a_ld, BLOCK_M);
  if (v != LCE_OK) return v;
  v = b_mn_major ? make_operand_tmap(&tb, dtype, true, b, n, k, b_ld, rows_of_b_tile(pair))
                 : make_operand_tmap(&tb, dtype, false, b, k, n, b_ld, rows_of_b_tile(pair));
  if (v != LCE_OK) return v;
  GemmParams gp;
  memset(&gp, 0, sizeof(gp));
  gp.m_tiles = (int)(m / BLOCK_M);
  gp.n_tiles = (int)(n / BLOCK_N);
  gp.splits = splits;
  gp.k_blocks = (int)(k / bk / splits);
  gp.raster_group = raster_group;
  gp.n_fastest = n_fastest ? 1 : 0;
  gp.out = out;
  gp.out_ld = n;
  gp.out_split_stride = m * n;
  gp.out_rows = (int)m;
  gp.out_cols = (int)n;
  gp.out_vector_ok = ((reinterpret_cast<uintptr_t>(out) & 31u) == 0) ? 1 : 0;
  gp.out_scale = 1.f;
  gp.status = dev_status;
  gp.clock_probe = reinterpret_cast<long long*>(dev_status + 2);
  CUtensorMap tc = ta;
  if (epilogue_tma_enabled() && (reinterpret_cast<uintptr_t>(out) & 15u) == 0) {
    if ((v = make_store_tmap(&tc, LCE_DTYPE_F32, out, n, (long long)splits * m, n)) != LCE_OK) return v;
    gp.out_tma = 1;
    gp.c_split_rows = (int)m;
  }
  cudaStream_t st = (cudaStream_t)stream;
  if (!a_mn_major && !b_mn_major)
    return launch_gemm_dtype<false, false, EPI_F32, false>(dtype, ta, tb, tc, gp, sms, st, pair);
  if (!a_mn_major && b_mn_major)
    return launch_gemm_dtype<false, true, EPI_F32, false>(dtype, ta, tb, tc, gp, sms, st, pair);
  if (a_mn_major && !b_mn_major)
    return launch_gemm_dtype<true, false, EPI_F32, false>(dtype, ta, tb, tc, gp, sms, st, pair);
  return launch_gemm_dtype<true, true, EPI_F32, false>(dtype, ta, tb, tc, gp, sms, st, pair);
}

}  // extern "C"

// ================================================================================================
// Loss evaluation without any caller-provided scratch (lce_eval_loss_static)
// ================================================================================================
namespace {

// Scratch of the allocation-free entry point. It lives in the library's device image, so every GPU that
// loads the library holds these 8 MiB until the process exits. In host code this name is only a handle
// for cudaGetSymbolAddress -- it is NOT a device address and must never be handed to a kernel as is.
static __device__ __align__(256) unsigned char g_static_scratch[LCE_STATIC_SCRATCH_BYTES];

std::mutex g_static_mutex;
void* g_static_scratch_ptr[kMaxDevices] = {};  // device address of g_static_scratch, per device

// Resolves (once per device, with that device current) the device address of the scratch array.
int static_scratch_address(void** out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return LCE_ERR_CUDA;
  if (dev < 0 || dev >= kMaxDevices) return LCE_ERR_UNSUPPORTED_DEVICE;
  std::lock_guard<std::mutex> lock(g_static_mutex);
  if (g_static_scratch_ptr[dev] == nullptr) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_static_scratch) != cudaSuccess || ptr == nullptr) return LCE_ERR_CUDA;
    g_static_scratch_ptr[dev] = ptr;
  }
  *out = g_static_scratch_ptr[dev];
  return LCE_OK;
}

}  // namespace

extern "C" int lce_eval_loss_static(const lce_problem* p_in, const void* x, int64_t x_ld, const void* weight,
                                    int64_t w_ld, const int64_t* labels, float* out5, void* stream) {
  if (p_in == nullptr || !x || !weight || !labels || !out5) return LCE_ERR_INVALID_ARGUMENT;
  // forward only, unsharded; the chunk length is chosen here so that everything fits the fixed scratch
  lce_problem p = *p_in;
  p.want_grad = 0;
  p.world = 1;
  p.vocab_offset = 0;
  p.chunk_buffers = 0;
  p.chunk_rows = BLOCK_M;  // provisional, for the shape checks
  int v = validate_problem(&p);
  if (v != LCE_OK) return v;
  const int sms = sm_count_or_default();
  long long best = 0;
  for (long long rows = BLOCK_M; rows <= round_up(p.n_rows_total, BLOCK_M); rows += BLOCK_M) {
    p.chunk_rows = rows;
    const size_t need = align_up(layout_workspace(&p, nullptr, sms).total, 256) + (size_t)ROW_PARTS * rows * sizeof(float);
    if (need > (size_t)LCE_STATIC_SCRATCH_BYTES) break;
    best = rows;
  }
  if (best == 0) return LCE_ERR_TOO_LARGE;  // even 128 rows of statistics exceed the fixed scratch: vocab too large
  // whole 256-row tiles when at least one fits: an even number of 128-row tiles runs on the CTA-pair kernel
  if (best >= 2 * BLOCK_M) best -= best % (2 * BLOCK_M);
  p.chunk_rows = best;

  void* scratch = nullptr;
  if ((v = static_scratch_address(&scratch)) != LCE_OK) return v;
  const size_t ws_bytes = align_up(layout_workspace(&p, nullptr, sms).total, 256);
  float* parts = reinterpret_cast<float*>(reinterpret_cast<char*>(scratch) + ws_bytes);

  // lce_begin clears every accumulator the pass sums into; all other scratch is written before it is read
  if ((v = lce_begin(&p, labels, scratch, stream)) != LCE_OK) return v;
  for (long long row0 = 0; row0 < p.n_rows_total; row0 += p.chunk_rows) {
    const long long rows = (p.n_rows_total - row0 < p.chunk_rows) ? p.n_rows_total - row0 : p.chunk_rows;
    if ((v = lce_forward_chunk(&p, x, x_ld, weight, w_ld, labels, row0, rows, scratch, parts, stream)) != LCE_OK)
      return v;
    if ((v = lce_combine_chunk(&p, parts, labels, row0, rows, scratch, stream)) != LCE_OK) return v;
  }
  return lce_finalize(&p, scratch, out5, stream);
}
