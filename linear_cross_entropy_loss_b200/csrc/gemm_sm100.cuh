// Persistent, warp-specialised tcgen05 GEMM engine for sm_100a.
//
//   D[M, N] = A[M, K] * B[N, K]^T        (fp32 accumulation in tensor memory)
//
// One CTA per SM walks a static list of 128 x 256 output tiles. Inside a CTA:
//   warp 0      TMA producer: fills a 4-deep ring of (A tile, B tile) K-blocks in shared memory
//   warp 1      MMA issuer:   one thread issues tcgen05.mma into one of two 256-column TMEM accumulators
//   warps 2..5  epilogue:     drain the other accumulator (thread <-> TMEM lane <-> output row)
// so that the epilogue of tile i overlaps the MMAs of tile i+1.
//
// Either operand may be K-major (K contiguous in global memory) or MN-major (M resp. N contiguous);
// this is what lets the three contractions of the loss
//   z  = x  * W        (A = x  K-major,  B = W  MN-major)      W is stored (H, V), V contiguous
//   dx = dZ * W^T      (A = dZ K-major,  B = W  K-major)
//   dW = x^T * dZ      (A = x  MN-major, B = dZ MN-major)
// run from the same buffers without ever materialising a transpose.
//
// Shared-memory operand tiles use the 128-byte swizzle that TMA writes and UMMA descriptors read:
//   K-major : row r (an M or N index) is 128 contiguous bytes of K at offset r * 128
//             (8-row groups 1024 bytes apart = stride byte offset)
//   MN-major: a TMA box is 128 bytes of MN x BLOCK_K rows of K (row k at offset k * 128; 8-row groups
//             1024 bytes apart = stride byte offset); consecutive boxes along MN are BLOCK_K * 128 bytes
//             apart (= leading byte offset). 32-bit MN-major operands use the 32-byte-atom variant of
//             the swizzle (4-row groups, 512 bytes apart).
#pragma once

#include "ptx.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace lce {

enum : int { KIND_F16 = 0, KIND_BF16 = 1, KIND_TF32 = 2 };
enum : int { EPI_F32 = 0, EPI_FWD = 1 };

constexpr int BLOCK_M = 128;
constexpr int BLOCK_N = 256;
constexpr int kStages = 4;
constexpr int kAccStages = 2;
constexpr int kTmemCols = 512;
constexpr int kGemmThreads = 192;
constexpr int kATileBytes = BLOCK_M * 128;  // 16 KiB
constexpr int kBTileBytes = BLOCK_N * 128;  // 32 KiB
constexpr int kStageBytes = kATileBytes + kBTileBytes;

// error codes written to the device status word
enum : int { DEV_OK = 0, DEV_WAIT_TIMEOUT_PRODUCER = 101, DEV_WAIT_TIMEOUT_MMA = 102, DEV_WAIT_TIMEOUT_EPILOGUE = 103 };

struct GemmShared {
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t acc_full[kAccStages];
  uint64_t acc_empty[kAccStages];
  uint32_t tmem_base;
  int abort_flag;
};

// Output staging for TMA stores: each of the four epilogue warps owns two buffers of 32 rows x 128 bytes
// (128-byte swizzle), filled from registers and drained by cp.async.bulk.tensor stores.
constexpr int kStoreStageBytes = 32 * 128;
constexpr int kStoreStagingBytes = 4 * 2 * kStoreStageBytes;  // 32 KiB per CTA

constexpr size_t kGemmSmemBytes =
    size_t(kStages) * kStageBytes + kStoreStagingBytes + 1024 /*alignment slack*/ + sizeof(GemmShared);

struct GemmParams {
  // tile grid; units = splits * n_tiles * m_tiles, walked in the order n_fastest selects
  int m_tiles;
  int n_tiles;
  int splits;
  int k_blocks;  // K-blocks (128 bytes of K each) per split
  int n_fastest; // 0: consecutive units walk M first (then N, then the K-split); 1: they walk N first
  int raster_group;  // kernels: 0 = walk the whole fast dimension, G > 0 = in bands of G tiles (unit_to_tile).
                     // Given to launch_gemm: 0 = the process default (chosen from the shape unless
                     // LCE_RASTER_GROUP says otherwise), -1 = no bands, -2 = chosen from the shape, G > 0 = bands of G
  // element offsets added to the tensor-map coordinates
  int a_mn0, a_k0, b_mn0, b_k0;

  // ---- EPI_F32: plain fp32 tile store / read-add-store
  float* out;
  long long out_ld;            // elements between output rows
  long long out_split_stride;  // elements between the outputs of consecutive K-splits
  int accumulate;              // 0: out = coef * acc, 1: out += coef * acc
  float out_scale;             // coef = out_scale / (*out_div)   (out_div may be null: coef = out_scale)
  const float* out_div;
  // ---- EPI_F32, 16-bit element types: accumulation across launches as a pair of arrays in the ELEMENT type,
  // sum = out_sum + out_res with out_sum = round(sum) and out_res = round(sum - out_sum) (about 16 significant
  // bits, against the 8 or 11 of the result). out_sum is the result itself after the last launch: no fp32
  // accumulator the size of the output, no conversion pass. `accumulate` = 0 for the first launch; out_res may be
  // null when nothing follows (last launch: the residual is not written) -- a single launch needs none at all.
  void* out_sum;
  void* out_res;
  long long out_pair_ld;       // elements between rows of out_sum and of out_res
  int out_pair_last;           // 1: last launch of the accumulation
  int out_rows;                // rows / columns of the output that exist; tiles may hang over both edges
  int out_cols;
  int out_vector_ok;           // 1: out (or out_sum / out_res) and their strides allow 32-byte accesses

  // ---- EPI_FWD: softmax statistics + exp slab
  void* slab;                  // [rows, slab_ld] in the input element type: exp(z - b) with b = the row's reference
                               // (row-reference mode) or the maximum of the (row, tile) (per-tile mode)
  long long slab_ld;
  int store_slab;              // 0 when no gradient is wanted
  float* tile_max;             // [n_tiles, stat_ld] per (V tile, row): max_j z
  float* tile_sum;             //                    sum_j exp(z - max)
  float* tile_ez;              //                    sum_j exp(z - max) * z      (monitoring)
  float* tile_sq;              //                    sum_j z^2                  (monitoring)
  long long stat_ld;
  float* target_logit;         // [rows] z[i, y_i], written by the one tile that holds column y_i
  const long long* labels;     // [rows_valid]
  int rows_valid;              // rows of this call that exist (the last 128-row tile may be partly padding)
  int cols_valid;              // vocabulary columns that exist (the last 256-column tile may be partly padding)
  long long ignore_index;
  long long vocab_offset;      // global class id of local column 0
  float scale;                 // logit scale (> 0)
  const float* row_ref;        // [rows] row-reference mode: slab = exp(z - row_ref[i]); null = reference 0

  // ---- EPI_F32: optional per-output-row factor (dx in row-reference mode: exp(ref - lse) (1 + 2 z_reg lse))
  const float* row_coef;

  // ---- all kernels: when non-null and *run_if == 0 the kernel returns at once (conditional re-run)
  const int* run_if;
  // ---- conditional re-run, finer: when non-null, a tile is skipped unless a flag is set for one of its
  // 256-row groups; group g covers rows [256 g, 256 g + 256) counted from row -run_mask_row0 of this call
  const int* run_mask;
  int run_mask_row0;

  // ---- output through shared memory and TMA (the third tensor map of the launch): EPI_FWD slab stores;
  // EPI_F32 tile stores of plain fp32 output that is only written (accumulate == 0, no element-type pair, no peer
  // scatter). The map describes exactly what exists, so TMA clips tiles at the edges.
  int out_tma;
  int c_row0;                  // row of the map that row 0 of this launch's output corresponds to
  int c_split_rows;            // EPI_F32: rows of the map between the outputs of consecutive K-splits

  int* status;                 // device status word (0 = ok)
  int tile_mode;               // forward epilogue: 1 = exp(z - tile max) even for bf16 / fp32
  long long* clock_probe;      // optional [2]: SM cycles and nanoseconds CTA 0 spent in the kernel (diagnostics)
  // EPI_F32 scatter mode (peer_rows_own > 0): the output rows are spread over the receive buffers of the ranks
  // that own them -- rank o owns chunk rows [o * peer_rows_own, (o + 1) * peer_rows_own) -- and split s of
  // this launch goes to slot peer_slot0 + s of the owner's buffer [slots][peer_rows_own][out_ld] at peer_out[o]
  float* peer_out[8];
  int peer_rows_own;           // multiple of BLOCK_M, so that a tile has one owner; 0 = plain output
  int peer_row0;               // chunk-local index of output row 0 of this launch
  int peer_slot0;
};

// --------------------------------------------------------------------------------------------------
// descriptors
// --------------------------------------------------------------------------------------------------
// Shared-memory matrix descriptor for a tile whose base is 1024-byte aligned.
// 16-bit operands and K-major tf32 use the plain 128-byte swizzle (16-byte chunks permuted over 8 rows).
// MN-major 32-bit operands exist in hardware only with the "128-byte swizzle, 32-byte atom" layout
// (32-byte chunks permuted over 4 rows), so there the K rows come in groups of 4 (512 bytes).
template <bool kMNMajor, int kBlockK, bool k32BitMN>
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr) {
  const uint64_t start = (smem_addr & 0x3FFFFu) >> 4;
  const uint64_t lbo = kMNMajor ? uint64_t((kBlockK * 128) >> 4) : 1ull;  // MN-major: next 128-byte MN box
  const uint64_t sbo = (k32BitMN ? 512ull : 1024ull) >> 4;                // next group of 8 (or 4) rows
  const uint64_t layout = k32BitMN ? 1ull /*SWIZZLE_128B_BASE32B*/ : 2ull /*SWIZZLE_128B*/;
  return start | (lbo << 16) | (sbo << 32) | (1ull << 46) /*descriptor version*/ | (layout << 61);
}

template <int kKind, bool kAMN, bool kBMN>
__host__ __device__ constexpr uint32_t make_instr_desc() {
  const uint32_t fmt = (kKind == KIND_F16) ? 0u : (kKind == KIND_BF16 ? 1u : 2u);
  return (1u << 4)                         // D format: f32
         | (fmt << 7) | (fmt << 10)        // A, B formats
         | ((kAMN ? 1u : 0u) << 15)        // A major: 0 = K, 1 = MN
         | ((kBMN ? 1u : 0u) << 16)        // B major
         | (uint32_t(BLOCK_N >> 3) << 17)  // N
         | (uint32_t(BLOCK_M >> 4) << 24); // M
}

// --------------------------------------------------------------------------------------------------
// epilogues (one thread = one output row of the 128 x 256 tile)
// --------------------------------------------------------------------------------------------------
template <int kKind>
struct SlabElem {
  using type = __half;
};
template <>
struct SlabElem<KIND_BF16> {
  using type = __nv_bfloat16;
};
template <>
struct SlabElem<KIND_TF32> {
  using type = float;
};

template <typename T>
__device__ __forceinline__ T cast_elem(float v);
template <>
__device__ __forceinline__ float cast_elem<float>(float v) { return v; }
template <>
__device__ __forceinline__ __half cast_elem<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 cast_elem<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// 32 consecutive elements of one output row, written as full 32-byte sectors (dst is 32-byte aligned).
__device__ __forceinline__ void store_slab_chunk(__half* dst, const float (&e)[32]) {
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    uint32_t v[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      __half2 h = __floats2half2_rn(e[16 * i + 2 * k], e[16 * i + 2 * k + 1]);
      v[k] = *reinterpret_cast<uint32_t*>(&h);
    }
    st_global_256(dst + 16 * i, v);
  }
}
__device__ __forceinline__ void store_slab_chunk(__nv_bfloat16* dst, const float (&e)[32]) {
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    uint32_t v[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      __nv_bfloat162 h = __floats2bfloat162_rn(e[16 * i + 2 * k], e[16 * i + 2 * k + 1]);
      v[k] = *reinterpret_cast<uint32_t*>(&h);
    }
    st_global_256(dst + 16 * i, v);
  }
}
__device__ __forceinline__ void store_slab_chunk(float* dst, const float (&e)[32]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint32_t v[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) v[k] = __float_as_uint(e[8 * i + k]);
    st_global_256(dst + 8 * i, v);
  }
}

// 32 consecutive 16-bit elements (64 bytes, 32-byte aligned) as floats.
__device__ __forceinline__ void load_elems32(const __nv_bfloat16* src, float (&f)[32]) {
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    uint32_t v[8];
    ld_global_256(src + 16 * i, v);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      f[16 * i + 2 * k] = __uint_as_float(v[k] << 16);
      f[16 * i + 2 * k + 1] = __uint_as_float(v[k] & 0xffff0000u);
    }
  }
}
__device__ __forceinline__ void load_elems32(const __half* src, float (&f)[32]) {
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    uint32_t v[8];
    ld_global_256(src + 16 * i, v);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float2 t = __half22float2(*reinterpret_cast<const __half2*>(&v[k]));
      f[16 * i + 2 * k] = t.x;
      f[16 * i + 2 * k + 1] = t.y;
    }
  }
}
__device__ __forceinline__ void load_elems32(const float* src, float (&f)[32]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint32_t v[8];
    ld_global_256(src + 8 * i, v);
#pragma unroll
    for (int k = 0; k < 8; ++k) f[8 * i + k] = __uint_as_float(v[k]);
  }
}
template <typename T>
__device__ __forceinline__ float elem_to_float(T v);
template <>
__device__ __forceinline__ float elem_to_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ float elem_to_float<__half>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float elem_to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

// One epilogue warp's pair of staging buffers. Lane l owns row l of the 32-row box: it writes its 128 bytes as eight
// 16-byte pieces (piece j lands at j ^ (l & 7), the 128-byte swizzle TMA expects), then lane 0 issues the store.
struct WarpStage {
  uint8_t* base;  // 2 * kStoreStageBytes, 1024-byte aligned
  int fills;      // boxes committed so far; selects the buffer

  // The buffer to fill next, once the store that last read it has finished reading (at most one newer store, the
  // one from the other buffer, may still be in flight).
  __device__ __forceinline__ uint8_t* acquire(int lane) {
    if (lane == 0) bulk_wait_group_read<1>();
    __syncwarp();
    return base + (fills & 1) * kStoreStageBytes;
  }
  static __device__ __forceinline__ void put(uint8_t* buf, int lane, int piece, uint32_t a, uint32_t b, uint32_t c,
                                             uint32_t d) {
    st_shared_128(buf + lane * 128 + ((piece ^ (lane & 7)) << 4), a, b, c, d);
  }
  // Stores the box whose first column is c0 and first row c1 of the tensor map.
  __device__ __forceinline__ void commit(const CUtensorMap* tm, const uint8_t* buf, int lane, int c0, int c1) {
    fence_proxy_async_smem();  // the generic-proxy writes above become visible to the TMA unit
    __syncwarp();
    if (lane == 0) {
      tma_store_2d(tm, buf, c0, c1);
      bulk_commit_group();
    }
    ++fills;
  }
  // Before the kernel ends: every store of this warp has been performed.
  __device__ __forceinline__ void drain(int lane) {
    if (lane == 0) bulk_wait_group<0>();
    __syncwarp();
  }
};

// 32 consecutive slab elements of this lane's row into the staging buffer: 16-bit types fill one half of the
// 128-byte row (pieces 4 * half .. 4 * half + 3), fp32 fills all of it.
__device__ __forceinline__ void stage_slab_chunk(__half*, uint8_t* buf, int lane, int half, const float (&e)[32]) {
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    uint32_t v[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      __half2 h = __floats2half2_rn(e[8 * q + 2 * k], e[8 * q + 2 * k + 1]);
      v[k] = *reinterpret_cast<uint32_t*>(&h);
    }
    WarpStage::put(buf, lane, 4 * half + q, v[0], v[1], v[2], v[3]);
  }
}
__device__ __forceinline__ void stage_slab_chunk(__nv_bfloat16*, uint8_t* buf, int lane, int half,
                                                 const float (&e)[32]) {
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    uint32_t v[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      __nv_bfloat162 h = __floats2bfloat162_rn(e[8 * q + 2 * k], e[8 * q + 2 * k + 1]);
      v[k] = *reinterpret_cast<uint32_t*>(&h);
    }
    WarpStage::put(buf, lane, 4 * half + q, v[0], v[1], v[2], v[3]);
  }
}
__device__ __forceinline__ void stage_slab_chunk(float*, uint8_t* buf, int lane, int /*half*/, const float (&e)[32]) {
#pragma unroll
  for (int q = 0; q < 8; ++q)
    WarpStage::put(buf, lane, q, __float_as_uint(e[4 * q]), __float_as_uint(e[4 * q + 1]),
                   __float_as_uint(e[4 * q + 2]), __float_as_uint(e[4 * q + 3]));
}

// Chunk c (32 columns) of a 256-column tile of the slab, through the staging buffers: two chunks of a 16-bit slab
// (one chunk of an fp32 slab) make one 128-byte-wide box of 32 rows.
template <typename Elem>
__device__ __forceinline__ void slab_chunk_via_tma(const GemmParams& p, const CUtensorMap* tmC, WarpStage& stage,
                                                   uint8_t*& buf, int lane, int c, int col0, int row0,
                                                   const float (&e)[32]) {
  constexpr bool kHalves = sizeof(Elem) == 2;
  if (!kHalves || (c & 1) == 0) buf = stage.acquire(lane);
  stage_slab_chunk(static_cast<Elem*>(nullptr), buf, lane, c & 1, e);
  if (!kHalves || (c & 1) == 1) stage.commit(tmC, buf, lane, col0 + (kHalves ? (c - 1) : c) * 32, row0);
}

// Forward epilogue. For its row i and this tile's 256 columns j (z = scale * acc):
//   tile_max = max_j z,  tile_sum = sum_j exp(z - tile_max),  slab[i, j] = exp(z - tile_max)
//   target_logit[i] = z[i, y_i] if column y_i lies in this tile
//   monitoring: tile_ez = sum_j exp(z - tile_max) * z,  tile_sq = sum_j z^2
// Two passes over the accumulator (max first). Used for fp16, whose narrow exponent range needs the
// exponentials normalised per tile; the slab is rescaled to the row's log-sum-exp afterwards.
template <int kKind, bool kMonitor>
__device__ __forceinline__ void epilogue_forward_tilemax(const GemmParams& p, const CUtensorMap* tmC, WarpStage& stage,
                                                         uint32_t taddr, int m_blk, int n_blk, int row_in_tile) {
  using Elem = typename SlabElem<kKind>::type;
  const long long r = (long long)m_blk * BLOCK_M + row_in_tile;
  const bool row_ok = r < p.rows_valid;                       // padding rows have no label and store no statistics
  const long long yv = row_ok ? p.labels[r] : p.ignore_index;
  const long long ycol_ll = yv - p.vocab_offset - (long long)n_blk * BLOCK_N;
  const int ycol = (yv != p.ignore_index && ycol_ll >= 0 && ycol_ll < BLOCK_N) ? (int)ycol_ll : -1;
  const int ncols = min(BLOCK_N, p.cols_valid - n_blk * BLOCK_N);  // columns of this tile that exist (>= 1)

  float mx = -INFINITY, sq = 0.f, tv = 0.f;
#pragma unroll 1
  for (int c = 0; c < BLOCK_N / 32; ++c) {
    uint32_t v[32];
    tmem_ld_32x32b_x32(taddr + c * 32, v);
    tmem_ld_wait();
    const int lim = ncols - c * 32;  // >= 32: the whole chunk exists
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      const float f = __uint_as_float(v[i]);
      if (i < lim) {
        mx = fmaxf(mx, f);
        if (kMonitor) sq = fmaf(f, f, sq);
      }
    }
    if ((ycol >> 5) == c) {
      const int sel = ycol & 31;
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (i == sel) tv = __uint_as_float(v[i]);
    }
  }

  const float sl2 = p.scale * 1.4426950408889634f;  // scale * log2(e)
  const float neg_m = -mx * sl2;
  float s = 0.f, ez = 0.f;
  Elem* slab_row = reinterpret_cast<Elem*>(p.slab) + r * p.slab_ld + (long long)n_blk * BLOCK_N;
  uint8_t* stage_buf = nullptr;
#pragma unroll 1
  for (int c = 0; c < BLOCK_N / 32; ++c) {
    uint32_t v[32];
    tmem_ld_32x32b_x32(taddr + c * 32, v);
    tmem_ld_wait();
    const int lim = ncols - c * 32;
    float e[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      const float f = __uint_as_float(v[i]);
      e[i] = (i < lim) ? fast_exp2(fmaf(f, sl2, neg_m)) : 0.f;  // padding columns hold 0 in the slab
      s += e[i];
      if (kMonitor && i < lim) ez = fmaf(e[i], f, ez);
    }
    if (p.store_slab) {
      if (p.out_tma)
        slab_chunk_via_tma<Elem>(p, tmC, stage, stage_buf, row_in_tile & 31, c, n_blk * BLOCK_N,
                                 p.c_row0 + m_blk * BLOCK_M + (row_in_tile & ~31), e);
      else
        store_slab_chunk(slab_row + c * 32, e);
    }
  }

  if (row_ok) {
    const long long si = (long long)n_blk * p.stat_ld + r;
    p.tile_max[si] = mx * p.scale;
    p.tile_sum[si] = s;
    if (kMonitor) {
      p.tile_ez[si] = ez * p.scale;
      p.tile_sq[si] = sq * p.scale * p.scale;
    }
    if (ycol >= 0) p.target_logit[r] = tv * p.scale;
  }
}

// Forward epilogue, row-reference mode (bf16 and fp32 slabs, whose exponent range is that of fp32): one pass.
//   slab[i, j] = exp(z - ref_i),  tile_sum = sum_j exp(z - ref_i),  tile_max = max_j z
//   monitoring: tile_ez = sum_j exp(z - ref_i) * z,  tile_sq = sum_j z^2
// ref_i is the same for every tile of row i (0 unless the pass is a re-run with ref_i = row max), so the tile
// sums of a row simply add up and dZ = exp(ref_i - lse_i) (1 + 2 z_reg lse_i) * slab - onehot needs only a
// PER-ROW factor: the slab feeds the gradient GEMMs as it is. If |row max - ref_i| turns out to exceed 60 the
// host-side sequence re-runs the chunk with ref_i = row max (see row_stats_rowref_kernel).
template <int kKind, bool kMonitor>
__device__ __forceinline__ void epilogue_forward_rowref(const GemmParams& p, const CUtensorMap* tmC, WarpStage& stage,
                                                        uint32_t taddr, int m_blk, int n_blk, int row_in_tile) {
  using Elem = typename SlabElem<kKind>::type;
  const long long r = (long long)m_blk * BLOCK_M + row_in_tile;
  const bool row_ok = r < p.rows_valid;                       // padding rows have no label and store no statistics
  const long long yv = row_ok ? p.labels[r] : p.ignore_index;
  const long long ycol_ll = yv - p.vocab_offset - (long long)n_blk * BLOCK_N;
  const int ycol = (yv != p.ignore_index && ycol_ll >= 0 && ycol_ll < BLOCK_N) ? (int)ycol_ll : -1;
  const int ncols = min(BLOCK_N, p.cols_valid - n_blk * BLOCK_N);  // columns of this tile that exist (>= 1)
  const float ref = (p.row_ref != nullptr && row_ok) ? p.row_ref[r] : 0.f;
  const float sl2 = p.scale * 1.4426950408889634f;  // scale * log2(e)
  const float neg_ref = -ref * 1.4426950408889634f;

  float mx = -INFINITY, s = 0.f, ez = 0.f, sq = 0.f, tv = 0.f;
  Elem* slab_row = reinterpret_cast<Elem*>(p.slab) + r * p.slab_ld + (long long)n_blk * BLOCK_N;
  uint8_t* stage_buf = nullptr;
#pragma unroll 1
  for (int c = 0; c < BLOCK_N / 32; ++c) {
    uint32_t v[32];
    tmem_ld_32x32b_x32(taddr + c * 32, v);
    tmem_ld_wait();
    const int lim = ncols - c * 32;  // >= 32: the whole chunk exists
    float e[32];
    if (lim >= 32) {
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const float f = __uint_as_float(v[i]);
        mx = fmaxf(mx, f);
        e[i] = fast_exp2(fmaf(f, sl2, neg_ref));
        s += e[i];
        if (kMonitor) {
          ez = fmaf(e[i], f, ez);
          sq = fmaf(f, f, sq);
        }
      }
    } else {  // chunk that hangs over the end of the vocabulary: padding columns count as exp(-inf) = 0
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const float f = __uint_as_float(v[i]);
        e[i] = 0.f;
        if (i < lim) {
          mx = fmaxf(mx, f);
          e[i] = fast_exp2(fmaf(f, sl2, neg_ref));
          s += e[i];
          if (kMonitor) {
            ez = fmaf(e[i], f, ez);
            sq = fmaf(f, f, sq);
          }
        }
      }
    }
    if ((ycol >> 5) == c) {
      const int sel = ycol & 31;
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (i == sel) tv = __uint_as_float(v[i]);
    }
    if (p.store_slab) {
      if (p.out_tma)
        slab_chunk_via_tma<Elem>(p, tmC, stage, stage_buf, row_in_tile & 31, c, n_blk * BLOCK_N,
                                 p.c_row0 + m_blk * BLOCK_M + (row_in_tile & ~31), e);
      else
        store_slab_chunk(slab_row + c * 32, e);
    }
  }

  if (row_ok) {
    const long long si = (long long)n_blk * p.stat_ld + r;
    p.tile_max[si] = mx * p.scale;
    p.tile_sum[si] = s;
    if (kMonitor) {
      p.tile_ez[si] = ez * p.scale;
      p.tile_sq[si] = sq * p.scale * p.scale;
    }
    if (ycol >= 0) p.target_logit[r] = tv * p.scale;
  }
}

// fp16 slabs are always normalised per tile; bf16 / fp32 slabs per row unless the launch asks for tiles.
template <int kKind>
struct ForwardMode {
  static constexpr bool kRowRef = (kKind != KIND_F16);
};

template <int kKind, bool kMonitor>
__device__ __forceinline__ void epilogue_forward(const GemmParams& p, const CUtensorMap* tmC, WarpStage& stage,
                                                 uint32_t taddr, int m_blk, int n_blk, int row_in_tile) {
  if (ForwardMode<kKind>::kRowRef && !p.tile_mode)
    epilogue_forward_rowref<kKind, kMonitor>(p, tmC, stage, taddr, m_blk, n_blk, row_in_tile);
  else
    epilogue_forward_tilemax<kKind, kMonitor>(p, tmC, stage, taddr, m_blk, n_blk, row_in_tile);
}

// Plain fp32 epilogue: result = coef * acc (+ what earlier launches accumulated). It goes to the fp32 array `out`
// (directly, through TMA, or scattered to peers), or -- out_sum given -- into the (sum, residual) pair of arrays in
// the input element type (see GemmParams).
template <int kKind>
__device__ __forceinline__ void epilogue_f32(const GemmParams& p, const CUtensorMap* tmC, WarpStage& stage,
                                             uint32_t taddr, int m_blk, int n_blk, int split, int row_in_tile) {
  using Elem = typename SlabElem<kKind>::type;
  const long long row = (long long)m_blk * BLOCK_M + row_in_tile;
  const bool row_ok = row < p.out_rows;
  const int ncols = min(BLOCK_N, p.out_cols - n_blk * BLOCK_N);  // columns of this tile that exist
  float* dst;
  if (p.peer_rows_own > 0) {
    const int chunk_row = p.peer_row0 + int(row);
    const int owner = min(chunk_row / p.peer_rows_own, 7);
    dst = p.peer_out[owner] +
          ((long long)(p.peer_slot0 + split) * p.peer_rows_own + (chunk_row - owner * p.peer_rows_own)) * p.out_ld +
          (long long)n_blk * BLOCK_N;
  } else {
    dst = p.out + (long long)split * p.out_split_stride + row * p.out_ld + (long long)n_blk * BLOCK_N;
  }
  const bool pair = p.out_sum != nullptr;
  Elem* dst_sum = reinterpret_cast<Elem*>(p.out_sum) + row * p.out_pair_ld + (long long)n_blk * BLOCK_N;
  Elem* dst_res = reinterpret_cast<Elem*>(p.out_res) + row * p.out_pair_ld + (long long)n_blk * BLOCK_N;
  const bool write_res = pair && p.out_res != nullptr && !p.out_pair_last;
  float coef = (p.out_div != nullptr) ? p.out_scale / __ldg(p.out_div) : p.out_scale;
  if (p.row_coef != nullptr) coef *= p.row_coef[row];  // row_coef covers the padded rows too
#pragma unroll 1
  for (int c = 0; c < BLOCK_N / 32; ++c) {
    uint32_t v[32];
    tmem_ld_32x32b_x32(taddr + c * 32, v);  // warp-collective: every lane takes part, even for rows that do not exist
    tmem_ld_wait();
    const int lim = ncols - c * 32;
    float r[32];
    if (p.out_tma) {
      // plain fp32 output that is only written: this warp's 32 rows x 32 columns go through shared memory and one
      // TMA store; TMA drops what lies outside the output
#pragma unroll
      for (int i = 0; i < 32; ++i) r[i] = coef * __uint_as_float(v[i]);
      const int lane = row_in_tile & 31;
      uint8_t* buf = stage.acquire(lane);
      stage_slab_chunk(static_cast<float*>(nullptr), buf, lane, 0, r);
      stage.commit(tmC, buf, lane, n_blk * BLOCK_N + c * 32,
                   p.c_row0 + split * p.c_split_rows + m_blk * BLOCK_M + (row_in_tile & ~31));
    } else if (p.peer_rows_own > 0) {
      // Scatter to the owning rank (whole padded tiles, so no masks). A thread holds 128 contiguous bytes of
      // ITS row, and storing them as they are gives 32 separate 32-byte segments per warp instruction, which a
      // link to another GPU carries poorly. So the four lanes of a group first exchange 32-byte units --
      // round t sends unit (q ^ t) to lane ^ t, after which lane q holds unit q of all four rows of its
      // group -- and then store row by row: each instruction writes 128 contiguous bytes of 8 rows.
#pragma unroll
      for (int i = 0; i < 32; ++i) r[i] = coef * __uint_as_float(v[i]);
      const int lane = row_in_tile & 31;
      const int q = lane & 3;
      float got[4][8];  // got[t] = unit q of row (lane ^ t)
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const int u = q ^ t;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const float lo = (u & 1) ? r[8 + k] : r[k];
          const float hi = (u & 1) ? r[24 + k] : r[16 + k];
          const float send = (u & 2) ? hi : lo;
          got[t][k] = (t == 0) ? send : __shfl_xor_sync(0xffffffffu, send, t);
        }
      }
      float* group_row0 = dst - (long long)q * p.out_ld + c * 32 + 8 * q;  // row (lane & ~3), this lane's unit
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int t = q ^ j;  // the round in which row (lane & ~3) + j arrived
        uint32_t o[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const float lo = (t & 1) ? got[1][k] : got[0][k];
          const float hi = (t & 1) ? got[3][k] : got[2][k];
          o[k] = __float_as_uint((t & 2) ? hi : lo);
        }
        st_global_256(group_row0 + (long long)j * p.out_ld, o);
      }
    } else if (!row_ok || lim <= 0) {
      // nothing of this chunk exists in the output
    } else if (pair && lim >= 32 && p.out_vector_ok) {
      // running sum and residual in the element type: sum = hi + lo + coef * acc; hi' = round(sum), lo' = round(sum - hi')
#pragma unroll
      for (int i = 0; i < 32; ++i) r[i] = coef * __uint_as_float(v[i]);
      if (p.accumulate) {
        float t[32];
        load_elems32(dst_sum + c * 32, t);
#pragma unroll
        for (int i = 0; i < 32; ++i) r[i] += t[i];
        load_elems32(dst_res + c * 32, t);
#pragma unroll
        for (int i = 0; i < 32; ++i) r[i] += t[i];
      }
      store_slab_chunk(dst_sum + c * 32, r);
      if (write_res) {
#pragma unroll
        for (int i = 0; i < 32; ++i) r[i] -= elem_to_float<Elem>(cast_elem<Elem>(r[i]));
        store_slab_chunk(dst_res + c * 32, r);
      }
    } else if (pair) {
      // edge of the output, or rows that are not 32-byte aligned: element by element
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        if (i < lim) {
          float val = coef * __uint_as_float(v[i]);
          if (p.accumulate) val += elem_to_float<Elem>(dst_sum[c * 32 + i]) + elem_to_float<Elem>(dst_res[c * 32 + i]);
          const Elem hi = cast_elem<Elem>(val);
          dst_sum[c * 32 + i] = hi;
          if (write_res) dst_res[c * 32 + i] = cast_elem<Elem>(val - elem_to_float<Elem>(hi));
        }
      }
    } else if (lim >= 32 && p.out_vector_ok) {
      // whole chunk inside the output and 32-byte accesses allowed
      if (p.accumulate) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          uint32_t o[8];
          ld_global_256(dst + c * 32 + 8 * i, o);
#pragma unroll
          for (int k = 0; k < 8; ++k)
            r[8 * i + k] = fmaf(coef, __uint_as_float(v[8 * i + k]), __uint_as_float(o[k]));
        }
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) r[i] = coef * __uint_as_float(v[i]);
      }
      store_slab_chunk(dst + c * 32, r);
    } else {
      // edge of the output, or an unaligned output: element by element
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        if (i < lim) {
          float val = coef * __uint_as_float(v[i]);
          if (p.accumulate) val += dst[c * 32 + i];
          dst[c * 32 + i] = val;
        }
      }
    }
    __syncwarp();  // the next TMEM load is warp-collective
  }
}

// True when the tile of `tile_rows` rows starting at row `row0` of this call takes part in the launch.
__device__ __forceinline__ bool tile_selected(const GemmParams& p, int row0, int tile_rows) {
  if (p.run_mask == nullptr) return true;
  const int first = (p.run_mask_row0 + row0) >> 8;
  const int last = (p.run_mask_row0 + row0 + tile_rows - 1) >> 8;
  int any = 0;
  for (int g = first; g <= last; ++g) any |= p.run_mask[g];
  return any != 0;
}

// Tile of the `rem`-th unit of one K-split. Without bands (raster_group == 0) the fast dimension -- M, or N when
// n_fastest -- is walked completely before the slow one advances, so the units in flight at one time cover the
// whole fast dimension times a few slow tiles. With raster_group = G the fast dimension is cut into bands of G
// tiles and each band is walked over the whole slow dimension before the next band starts: the units in flight
// form a block of about G x (CTAs / G) tiles. When the fast dimension is long this block shares more operand rows
// per byte fetched, and less of the band's operand (G tiles x K) is fetched from DRAM again for every slow tile.
__device__ __forceinline__ void unit_to_tile(const GemmParams& p, int rem, int& m_blk, int& n_blk) {
  const int nf = p.n_fastest ? p.n_tiles : p.m_tiles;
  int f, s;
  if (p.raster_group <= 0 || p.raster_group >= nf) {
    s = rem / nf;
    f = rem - s * nf;
  } else {
    const int ns = p.n_fastest ? p.m_tiles : p.n_tiles;
    const int per_band = p.raster_group * ns;  // the last band may be narrower; it is the only one
    const int band = rem / per_band;
    const int r = rem - band * per_band;
    const int f0 = band * p.raster_group;
    const int width = min(p.raster_group, nf - f0);
    s = r / width;
    f = f0 + (r - s * width);
  }
  m_blk = p.n_fastest ? s : f;
  n_blk = p.n_fastest ? f : s;
}

// --------------------------------------------------------------------------------------------------
// the kernel
// --------------------------------------------------------------------------------------------------
template <int kKind, bool kAMN, bool kBMN, int kEpi, bool kMonitor>
__global__ void __launch_bounds__(kGemmThreads, 1)
lce_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                const __grid_constant__ CUtensorMap tmC, const GemmParams p) {
  constexpr int ES = (kKind == KIND_TF32) ? 4 : 2;  // operand element size in bytes
  constexpr int BLOCK_K = 128 / ES;                 // elements of K per 128-byte swizzle row
  constexpr int UMMA_K = 32 / ES;                   // K elements per tcgen05.mma
  constexpr int MN_BOX = 128 / ES;                  // elements of MN per MN-major TMA box
  constexpr int K_STEPS = BLOCK_K / UMMA_K;         // 4
  // descriptor start-address advance (16-byte units) per UMMA_K step
  constexpr uint32_t kAdvA = kAMN ? (UMMA_K * 128) >> 4 : 32 >> 4;
  constexpr uint32_t kAdvB = kBMN ? (UMMA_K * 128) >> 4 : 32 >> 4;
  constexpr uint32_t kIdesc = make_instr_desc<kKind, kAMN, kBMN>();

  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* staging = tiles + size_t(kStages) * kStageBytes;  // 1024-byte aligned: the ring is a multiple of 1024 bytes
  GemmShared* sh = reinterpret_cast<GemmShared*>(staging + kStoreStagingBytes);
  volatile int* abort_flag = &sh->abort_flag;
  if (p.run_if != nullptr && *p.run_if == 0) return;  // uniform over the grid: nothing has been set up yet

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&sh->full[s], 1);
      mbar_init(&sh->empty[s], 1);
    }
    for (int a = 0; a < kAccStages; ++a) {
      mbar_init(&sh->acc_full[a], 1);
      mbar_init(&sh->acc_empty[a], 4);  // one arrival per epilogue warp
    }
    sh->abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    tma_prefetch_desc(&tmC);
  }
  if (warp == 1) {
    tmem_alloc(&sh->tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = sh->tmem_base;
  long long probe_c0 = 0, probe_t0 = 0;
  if (p.clock_probe != nullptr && blockIdx.x == 0 && threadIdx.x == 64) {
    probe_c0 = clock64();
    probe_t0 = (long long)global_timer_ns();
  }

  const int units = p.splits * p.n_tiles * p.m_tiles;
  const int tiles_mn = p.n_tiles * p.m_tiles;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int unit = blockIdx.x; ok && unit < units; unit += gridDim.x) {
        const int split = unit / tiles_mn;
        const int rem = unit - split * tiles_mn;
        int m_blk, n_blk;
        unit_to_tile(p, rem, m_blk, n_blk);
        const int a_mn = p.a_mn0 + m_blk * BLOCK_M;
        const int b_mn = p.b_mn0 + n_blk * BLOCK_N;
        if (!tile_selected(p, m_blk * BLOCK_M, BLOCK_M)) continue;
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(&sh->empty[stage], phase ^ 1u, abort_flag)) {
            atomicCAS(p.status, DEV_OK, DEV_WAIT_TIMEOUT_PRODUCER);
            ok = false;
            break;
          }
          uint8_t* sA = tiles + size_t(stage) * kStageBytes;
          uint8_t* sB = sA + kATileBytes;
          const int kc = (split * p.k_blocks + kb) * BLOCK_K;
          mbar_arrive_expect_tx(&sh->full[stage], kStageBytes);
          if (!kAMN) {
            tma_load_2d(sA, &tmA, &sh->full[stage], p.a_k0 + kc, a_mn);
          } else {
#pragma unroll
            for (int j = 0; j < BLOCK_M / MN_BOX; ++j)
              tma_load_2d(sA + j * (BLOCK_K * 128), &tmA, &sh->full[stage], a_mn + j * MN_BOX, p.a_k0 + kc);
          }
          if (!kBMN) {
            tma_load_2d(sB, &tmB, &sh->full[stage], p.b_k0 + kc, b_mn);
          } else {
#pragma unroll
            for (int j = 0; j < BLOCK_N / MN_BOX; ++j)
              tma_load_2d(sB + j * (BLOCK_K * 128), &tmB, &sh->full[stage], b_mn + j * MN_BOX, p.b_k0 + kc);
          }
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int unit = blockIdx.x; ok && unit < units; unit += gridDim.x) {
        if (p.run_mask != nullptr) {  // same tile selection as the producer and the epilogue warps
          const int rem = unit % tiles_mn;
          int m_sel, n_sel;
          unit_to_tile(p, rem, m_sel, n_sel);
          if (!tile_selected(p, m_sel * BLOCK_M, BLOCK_M)) continue;
        }
        if (!mbar_wait(&sh->acc_empty[acc], acc_phase ^ 1u, abort_flag)) {
          atomicCAS(p.status, DEV_OK, DEV_WAIT_TIMEOUT_MMA);
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + uint32_t(acc * BLOCK_N);
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(&sh->full[stage], phase, abort_flag)) {
            atomicCAS(p.status, DEV_OK, DEV_WAIT_TIMEOUT_MMA);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t sA = smem_u32(tiles + size_t(stage) * kStageBytes);
          const uint64_t adesc = make_smem_desc<kAMN, BLOCK_K, kAMN && kKind == KIND_TF32>(sA);
          const uint64_t bdesc = make_smem_desc<kBMN, BLOCK_K, kBMN && kKind == KIND_TF32>(sA + kATileBytes);
#pragma unroll
          for (int k = 0; k < K_STEPS; ++k) {
            const uint32_t accum = (kb | k) != 0 ? 1u : 0u;
            if (kKind == KIND_TF32)
              umma_tf32(d_tmem, adesc + uint64_t(k * kAdvA), bdesc + uint64_t(k * kAdvB), kIdesc, accum);
            else
              umma_f16(d_tmem, adesc + uint64_t(k * kAdvA), bdesc + uint64_t(k * kAdvB), kIdesc, accum);
          }
          umma_commit(&sh->empty[stage]);  // frees the smem stage once these MMAs have read it
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        umma_commit(&sh->acc_full[acc]);  // accumulator complete -> epilogue
        if (++acc == kAccStages) {
          acc = 0;
          acc_phase ^= 1u;
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue warps
    const int lane_group = warp & 3;  // a warp may only touch TMEM lanes [32 * (warp % 4), +32)
    const int row_in_tile = lane_group * 32 + lane;
    WarpStage stage{staging + lane_group * 2 * kStoreStageBytes, 0};
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int unit = blockIdx.x; unit < units; unit += gridDim.x) {
      const int split = unit / tiles_mn;
      const int rem = unit - split * tiles_mn;
      int m_blk, n_blk;
      unit_to_tile(p, rem, m_blk, n_blk);
      if (!tile_selected(p, m_blk * BLOCK_M, BLOCK_M)) continue;
      if (!mbar_wait_warp(&sh->acc_full[acc], acc_phase, abort_flag)) {
        if (lane == 0) atomicCAS(p.status, DEV_OK, DEV_WAIT_TIMEOUT_EPILOGUE);
        break;
      }
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + (uint32_t(lane_group * 32) << 16) + uint32_t(acc * BLOCK_N);
      if (kEpi == EPI_FWD)
        epilogue_forward<kKind, kMonitor>(p, &tmC, stage, taddr, m_blk, n_blk, row_in_tile);
      else
        epilogue_f32<kKind>(p, &tmC, stage, taddr, m_blk, n_blk, split, row_in_tile);
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh->acc_empty[acc]);
      if (++acc == kAccStages) {
        acc = 0;
        acc_phase ^= 1u;
      }
    }
    stage.drain(lane);  // this warp's TMA stores have been performed before the CTA's shared memory goes away
  }

  // ------------------------------------------------------------------ teardown
  if (p.clock_probe != nullptr && blockIdx.x == 0 && threadIdx.x == 64) {
    p.clock_probe[0] = clock64() - probe_c0;
    p.clock_probe[1] = (long long)global_timer_ns() - probe_t0;
  }
  if (*abort_flag != 0) {
    // a wait ran out: give copies that may still be in flight time to land before smem goes away
    for (int i = 0; i < 64; ++i) __nanosleep(10000);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// --------------------------------------------------------------------------------------------------
// CTA-pair variant (cta_group::2): two CTAs of a cluster share one 256 x 256 output tile.
//
// CTA r of the pair owns accumulator rows [128 r, 128 r + 128) of the tile in its own TMEM, loads the
// matching 128 rows of A and columns [128 r, 128 r + 128) of B into its own shared memory, and runs its
// own epilogue; CTA 0 alone issues the MMAs, which read both CTAs' operand tiles. Per K-block each SM
// therefore stages and reads 32 KiB instead of 48 KiB, which is what lets the tensor pipes run closer
// to their peak under the chip's power limit.
//
// Barriers: every TMA load of either CTA counts its bytes on CTA 0's full[stage]; CTA 0 commits each
// MMA batch to empty[stage] of BOTH CTAs (one commit instruction addressed to both) and each finished
// accumulator to acc_full of both; the epilogue
// warps of both CTAs arrive on CTA 0's acc_empty (8 arrivals).
// --------------------------------------------------------------------------------------------------
constexpr int kPairStages = 6;
constexpr int kPairBTileBytes = (BLOCK_N / 2) * 128;  // 16 KiB: this CTA's half of the B tile
constexpr int kPairStageBytes = kATileBytes + kPairBTileBytes;
constexpr int PAIR_M = 2 * BLOCK_M;

struct GemmPairShared {
  uint64_t full[kPairStages];
  uint64_t empty[kPairStages];
  uint64_t acc_full[kAccStages];
  uint64_t acc_empty[kAccStages];
  uint32_t tmem_base;
  int abort_flag;
};

constexpr size_t kGemmPairSmemBytes =
    size_t(kPairStages) * kPairStageBytes + kStoreStagingBytes + 1024 + sizeof(GemmPairShared);
static_assert(kGemmPairSmemBytes <= 232448, "dynamic shared memory limit of sm_100");

template <int kKind, bool kAMN, bool kBMN>
__host__ __device__ constexpr uint32_t make_instr_desc_pair() {
  const uint32_t fmt = (kKind == KIND_F16) ? 0u : (kKind == KIND_BF16 ? 1u : 2u);
  return (1u << 4) | (fmt << 7) | (fmt << 10) | ((kAMN ? 1u : 0u) << 15) | ((kBMN ? 1u : 0u) << 16) |
         (uint32_t(BLOCK_N >> 3) << 17) | (uint32_t(PAIR_M >> 4) << 24);
}

// p.m_tiles counts 256-row tiles here.
template <int kKind, bool kAMN, bool kBMN, int kEpi, bool kMonitor>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
lce_gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                     const __grid_constant__ CUtensorMap tmC, const GemmParams p) {
  constexpr int ES = (kKind == KIND_TF32) ? 4 : 2;
  constexpr int BLOCK_K = 128 / ES;
  constexpr int UMMA_K = 32 / ES;
  constexpr int MN_BOX = 128 / ES;
  constexpr int K_STEPS = BLOCK_K / UMMA_K;
  constexpr uint32_t kAdvA = kAMN ? (UMMA_K * 128) >> 4 : 32 >> 4;
  constexpr uint32_t kAdvB = kBMN ? (UMMA_K * 128) >> 4 : 32 >> 4;
  constexpr uint32_t kIdesc = make_instr_desc_pair<kKind, kAMN, kBMN>();
  constexpr int HALF_N = BLOCK_N / 2;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* staging = tiles + size_t(kPairStages) * kPairStageBytes;  // 1024-byte aligned: the ring is a multiple of 1024 bytes
  GemmPairShared* sh = reinterpret_cast<GemmPairShared*>(staging + kStoreStagingBytes);
  volatile int* abort_flag = &sh->abort_flag;
  if (p.run_if != nullptr && *p.run_if == 0) return;  // uniform over the grid: nothing has been set up yet

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = (rank == 0);
  const int cluster_id = blockIdx.x >> 1;
  const int n_clusters = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kPairStages; ++s) {
      mbar_init(&sh->full[s], 1);   // used in CTA 0 only: one expect_tx arrival + the bytes of both CTAs
      mbar_init(&sh->empty[s], 1);  // one commit from CTA 0
    }
    for (int a = 0; a < kAccStages; ++a) {
      mbar_init(&sh->acc_full[a], 1);
      mbar_init(&sh->acc_empty[a], 8);  // used in CTA 0 only: 4 epilogue warps of each CTA
    }
    sh->abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    tma_prefetch_desc(&tmC);
  }
  if (warp == 1) {
    tmem_alloc_pair(&sh->tmem_base, kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  cluster_sync_all();  // both CTAs' barriers are initialised and both allocations are done
  tc_fence_after_sync();
  const uint32_t tmem_base = sh->tmem_base;
  long long probe_c0 = 0, probe_t0 = 0;
  if (p.clock_probe != nullptr && blockIdx.x == 0 && threadIdx.x == 64) {
    probe_c0 = clock64();
    probe_t0 = (long long)global_timer_ns();
  }

  const int units = p.splits * p.n_tiles * p.m_tiles;
  const int tiles_mn = p.n_tiles * p.m_tiles;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int unit = cluster_id; ok && unit < units; unit += n_clusters) {
        const int split = unit / tiles_mn;
        const int rem = unit - split * tiles_mn;
        int m_blk, n_blk;
        unit_to_tile(p, rem, m_blk, n_blk);
        const int a_mn = p.a_mn0 + m_blk * PAIR_M + int(rank) * BLOCK_M;
        const int b_mn = p.b_mn0 + n_blk * BLOCK_N + int(rank) * HALF_N;
        if (!tile_selected(p, m_blk * PAIR_M, PAIR_M)) continue;
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(&sh->empty[stage], phase ^ 1u, abort_flag)) {
            atomicCAS(p.status, DEV_OK, DEV_WAIT_TIMEOUT_PRODUCER);
            ok = false;
            break;
          }
          uint8_t* sA = tiles + size_t(stage) * kPairStageBytes;
          uint8_t* sB = sA + kATileBytes;
          const int kc = (split * p.k_blocks + kb) * BLOCK_K;
          if (leader) mbar_arrive_expect_tx(&sh->full[stage], 2 * kPairStageBytes);
          const uint32_t full0 = map_to_cta(smem_u32(&sh->full[stage]), 0);
          if (!kAMN) {
            tma_load_2d_pair(sA, &tmA, full0, p.a_k0 + kc, a_mn);
          } else {
#pragma unroll
            for (int j = 0; j < BLOCK_M / MN_BOX; ++j)
              tma_load_2d_pair(sA + j * (BLOCK_K * 128), &tmA, full0, a_mn + j * MN_BOX, p.a_k0 + kc);
          }
          if (!kBMN) {
            tma_load_2d_pair(sB, &tmB, full0, p.b_k0 + kc, b_mn);
          } else {
#pragma unroll
            for (int j = 0; j < HALF_N / MN_BOX; ++j)
              tma_load_2d_pair(sB + j * (BLOCK_K * 128), &tmB, full0, b_mn + j * MN_BOX, p.b_k0 + kc);
          }
          if (++stage == kPairStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (CTA 0 only)
    if (leader && lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int unit = cluster_id; ok && unit < units; unit += n_clusters) {
        if (p.run_mask != nullptr) {  // same tile selection as the producers and the epilogue warps
          const int rem = unit % tiles_mn;
          int m_sel, n_sel;
          unit_to_tile(p, rem, m_sel, n_sel);
          if (!tile_selected(p, m_sel * PAIR_M, PAIR_M)) continue;
        }
        if (!mbar_wait(&sh->acc_empty[acc], acc_phase ^ 1u, abort_flag)) {
          atomicCAS(p.status, DEV_OK, DEV_WAIT_TIMEOUT_MMA);
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + uint32_t(acc * BLOCK_N);
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(&sh->full[stage], phase, abort_flag)) {
            atomicCAS(p.status, DEV_OK, DEV_WAIT_TIMEOUT_MMA);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t sA = smem_u32(tiles + size_t(stage) * kPairStageBytes);
          const uint64_t adesc = make_smem_desc<kAMN, BLOCK_K, kAMN && kKind == KIND_TF32>(sA);
          const uint64_t bdesc = make_smem_desc<kBMN, BLOCK_K, kBMN && kKind == KIND_TF32>(sA + kATileBytes);
#pragma unroll
          for (int k = 0; k < K_STEPS; ++k) {
            const uint32_t accum = (kb | k) != 0 ? 1u : 0u;
            if (kKind == KIND_TF32)
              umma_pair_tf32(d_tmem, adesc + uint64_t(k * kAdvA), bdesc + uint64_t(k * kAdvB), kIdesc, accum);
            else
              umma_pair_f16(d_tmem, adesc + uint64_t(k * kAdvA), bdesc + uint64_t(k * kAdvB), kIdesc, accum);
          }
          const uint32_t e_local = smem_u32(&sh->empty[stage]);
          // one commit that arrives on empty[stage] of both CTAs (two separate commits cost 4 % of the
          // tensor pipe's time: the issuing thread is on the critical path)
          umma_pair_commit_both(e_local);
          if (++stage == kPairStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        umma_pair_commit_both(smem_u32(&sh->acc_full[acc]));
        if (++acc == kAccStages) {
          acc = 0;
          acc_phase ^= 1u;
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue warps (both CTAs)
    const int lane_group = warp & 3;
    const int row_in_tile = lane_group * 32 + lane;
    WarpStage stage{staging + lane_group * 2 * kStoreStageBytes, 0};
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int unit = cluster_id; unit < units; unit += n_clusters) {
      const int split = unit / tiles_mn;
      const int rem = unit - split * tiles_mn;
      int m_blk, n_blk;
      unit_to_tile(p, rem, m_blk, n_blk);
      const int m_blk128 = m_blk * 2 + int(rank);  // this CTA's 128-row block
      if (!tile_selected(p, m_blk * PAIR_M, PAIR_M)) continue;
      if (!mbar_wait_warp(&sh->acc_full[acc], acc_phase, abort_flag)) {
        if (lane == 0) atomicCAS(p.status, DEV_OK, DEV_WAIT_TIMEOUT_EPILOGUE);
        break;
      }
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + (uint32_t(lane_group * 32) << 16) + uint32_t(acc * BLOCK_N);
      if (kEpi == EPI_FWD)
        epilogue_forward<kKind, kMonitor>(p, &tmC, stage, taddr, m_blk128, n_blk, row_in_tile);
      else
        epilogue_f32<kKind>(p, &tmC, stage, taddr, m_blk128, n_blk, split, row_in_tile);
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&sh->acc_empty[acc]), 0));
      if (++acc == kAccStages) {
        acc = 0;
        acc_phase ^= 1u;
      }
    }
    stage.drain(lane);
  }

  // ------------------------------------------------------------------ teardown
  if (p.clock_probe != nullptr && blockIdx.x == 0 && threadIdx.x == 64) {
    p.clock_probe[0] = clock64() - probe_c0;
    p.clock_probe[1] = (long long)global_timer_ns() - probe_t0;
  }
  if (*abort_flag != 0) {
    for (int i = 0; i < 64; ++i) __nanosleep(10000);
  }
  tc_fence_before_sync();
  __syncwarp();
  cluster_sync_all();  // neither CTA may leave while the peer can still touch its shared memory or TMEM
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

}  // namespace lce
