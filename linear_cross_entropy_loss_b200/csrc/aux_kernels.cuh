// Memory-bound helper kernels around the three tensor-core contractions:
//   begin_kernel        count valid labels, clear the pass accumulators
//   row_stats_kernel    per row: merge the per-V-tile (max, sumexp, ...) into one partial per rank
//   combine_kernel      per row: merge the ranks' partials -> log-sum-exp; accumulate loss/metric sums
//   dz_transform_kernel slab: exp(z - tile max) -> dZ = softmax * (1 + 2 z_reg lse) - onehot, in place
//   dx_reduce_kernel    sum the K-split partials of dx in a fixed order, cast
//   finalize_kernel     the five output scalars
//   scale_cast_kernel   grad * factor with a type conversion
// All reductions run in a fixed order (no atomics), so results are bitwise reproducible.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cstdint>

namespace lce {

struct PassScalars {
  double sum_nll;    // sum over valid rows of (lse - target logit)
  double sum_lse2;   // sum over valid rows of lse^2
  double sum_ent;    // sum over valid rows of softmax entropy
  double sum_norm;   // sum over ALL rows of ||z_i||_2
  float max_logit;   // max over ALL rows and columns of z
  float n_valid;     // number of rows whose label is not ignore_index
  int status;        // device status word, 0 = ok
  int unused0;
  int rerun_groups;  // row-reference mode: 256-row groups of this pass whose forward had to be recomputed ...
  int seen_groups;   // ... out of this many (what a caller needs to pick the slab mode of its next pass)
};

// Per-row partials a rank exports per chunk:
//   [0] base b (the reference the sums are relative to), [1] sum_j exp(z - b), [2] target logit (0 if not owned),
//   [3] sum_j exp(z - b) z, [4] sum_j z^2, [5] max_j z
constexpr int ROW_PARTS = 6;
// Row-reference mode keeps exp(z - ref_i) in fp32 / bf16: finite row sums need (row max - ref_i) below about
// 88 - ln(V), and the entries that matter (within ~25 of the row max) need it above about -60. Outside
// [-kRefBelow, kRefAbove] the forward of the chunk is re-run with ref_i = row max.
constexpr float kRefAbove = 72.f;
constexpr float kRefBelow = 60.f;
// The first forward takes ref_i = (max logit over the first kProbeTiles vocabulary tiles) + kProbeMargin: the
// probe maximum never exceeds the row maximum, so the margin centres the window on the gap between the two
// (gaps of -2 .. 130 pass: logits with a standard deviation up to about 45 at V = 131072).
constexpr int kProbeTiles = 2;
constexpr float kProbeMargin = 58.f;

// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ double block_sum_double(double v, double* scratch /*[32]*/) {
  for (int o = 16; o > 0; o >>= 1) v += __shfl_down_sync(0xffffffffu, v, o);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  double t = 0.0;
  if (warp == 0) {
    t = (lane < (blockDim.x >> 5)) ? scratch[lane] : 0.0;
    for (int o = 16; o > 0; o >>= 1) t += __shfl_down_sync(0xffffffffu, t, o);
  }
  return t;  // valid in thread 0
}
__device__ __forceinline__ float block_max_float(float v, float* scratch /*[32]*/) {
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_down_sync(0xffffffffu, v, o));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = -INFINITY;
  if (warp == 0) {
    t = (lane < (blockDim.x >> 5)) ? scratch[lane] : -INFINITY;
    for (int o = 16; o > 0; o >>= 1) t = fmaxf(t, __shfl_down_sync(0xffffffffu, t, o));
  }
  return t;
}

// One block. Counts labels != ignore_index and resets the accumulators of the pass.
// rescue_groups / rescue_groups2: the re-run flags of the workspace's one or two sets of per-chunk buffers
// (n_groups ints each: one per 256-row group, then the "any group flagged" word of the chunk).
__global__ void begin_kernel(const long long* __restrict__ labels, long long n, long long ignore_index,
                             PassScalars* sc, int* rescue_groups, int* rescue_groups2, int n_groups) {
  for (int g = threadIdx.x; g < n_groups; g += blockDim.x) {
    rescue_groups[g] = 0;
    if (rescue_groups2 != nullptr) rescue_groups2[g] = 0;
  }
  __shared__ double scratch[32];
  double cnt = 0.0;
  for (long long i = threadIdx.x; i < n; i += blockDim.x) cnt += (labels[i] != ignore_index) ? 1.0 : 0.0;
  const double total = block_sum_double(cnt, scratch);
  if (threadIdx.x == 0) {
    sc->sum_nll = 0.0;
    sc->sum_lse2 = 0.0;
    sc->sum_ent = 0.0;
    sc->sum_norm = 0.0;
    sc->max_logit = -INFINITY;
    sc->n_valid = (float)total;
    sc->status = 0;
    sc->unused0 = 0;
    sc->rerun_groups = 0;
    sc->seen_groups = 0;
  }
}

// Merges (m2, s2, u2) into the running (m, s, u):  s = sum exp(z - m),  u = sum exp(z - m) * z.
__device__ __forceinline__ void lse_merge(float& m, float& s, float& u, float m2, float s2, float u2) {
  if (m2 > m) {
    const float f = __expf(m - m2);  // m = -inf on the first merge -> f = 0
    s = s * f + s2;
    u = u * f + u2;
    m = m2;
  } else {
    const float f = __expf(m2 - m);
    s += s2 * f;
    u += u2 * f;
  }
}

// Block = 32 rows x 8 warps; warp w walks V tiles w, w+8, ...; lane = row. Per-tile statistics are
// stored [tile][row], so each warp load is 128 contiguous bytes.
// parts layout: [ROW_PARTS][stat_ld].
template <bool kMonitor>
__global__ void __launch_bounds__(256)
row_stats_kernel(const float* __restrict__ tile_max, const float* __restrict__ tile_sum,
                 const float* __restrict__ tile_ez, const float* __restrict__ tile_sq,
                 const float* __restrict__ target_logit, const long long* __restrict__ labels, int rows,
                 int n_tiles, long long stat_ld, long long ignore_index, long long vocab_offset,
                 long long vocab_local, float* __restrict__ parts) {
  __shared__ float sm[8][4][32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = blockIdx.x * 32 + lane;
  float m = -INFINITY, s = 0.f, u = 0.f, q = 0.f;
  if (r < rows) {
    for (int t = warp; t < n_tiles; t += 8) {
      const long long i = (long long)t * stat_ld + r;
      const float mt = tile_max[i], st = tile_sum[i];
      const float ut = kMonitor ? tile_ez[i] : 0.f;
      if (kMonitor) q += tile_sq[i];
      lse_merge(m, s, u, mt, st, ut);
    }
  }
  sm[warp][0][lane] = m;
  sm[warp][1][lane] = s;
  sm[warp][2][lane] = u;
  sm[warp][3][lane] = q;
  __syncthreads();
  if (warp == 0 && r < rows) {
    for (int w = 1; w < 8; ++w) {
      lse_merge(m, s, u, sm[w][0][lane], sm[w][1][lane], sm[w][2][lane]);
      q += sm[w][3][lane];
    }
    const long long yv = labels[r];
    const long long yl = yv - vocab_offset;
    const bool own = (yv != ignore_index) && yl >= 0 && yl < vocab_local;
    parts[0 * stat_ld + r] = m;
    parts[1 * stat_ld + r] = s;
    parts[2 * stat_ld + r] = own ? target_logit[r] : 0.f;
    parts[3 * stat_ld + r] = u;
    parts[4 * stat_ld + r] = q;
    parts[5 * stat_ld + r] = m;
  }
}

// Row-reference mode: all tiles of a row share the reference ref_i (0, or row_ref[i] in a re-run), so the
// per-tile sums add up. Same thread layout as row_stats_kernel. Also writes row_ref_out[i] = row max (the
// reference a re-run would use), row_base_out[i] = ref_i, and raises *rescue when row max - ref_i leaves
// [-kRefBelow, kRefAbove].
// run_if: when non-null and 0 the kernel does nothing (it belongs to a conditional re-run).
template <bool kMonitor>
__global__ void __launch_bounds__(256)
row_stats_rowref_kernel(const float* __restrict__ tile_max, const float* __restrict__ tile_sum,
                        const float* __restrict__ tile_ez, const float* __restrict__ tile_sq,
                        const float* __restrict__ target_logit, const long long* __restrict__ labels, int rows,
                        int n_tiles, long long stat_ld, long long ignore_index, long long vocab_offset,
                        long long vocab_local, const float* row_ref_in, float* row_ref_out, float* row_base_out,
                        int* rescue, int* rescue_groups, int group_row0, const int* run_if,
                        float* __restrict__ parts) {
  // rescue_groups[g]: set when a row of the 256-row group g (rows counted from -group_row0) needs the re-run.
  // In the re-run itself (run_if given) only the flagged groups were recomputed, so only they are re-read.
  if (run_if != nullptr && (*run_if == 0 || rescue_groups[(group_row0 + blockIdx.x * 32) >> 8] == 0)) return;
  __shared__ float sm[8][4][32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = blockIdx.x * 32 + lane;
  float m = -INFINITY, s = 0.f, u = 0.f, q = 0.f;
  if (r < rows) {
    for (int t = warp; t < n_tiles; t += 8) {
      const long long i = (long long)t * stat_ld + r;
      m = fmaxf(m, tile_max[i]);
      s += tile_sum[i];
      if (kMonitor) {
        u += tile_ez[i];
        q += tile_sq[i];
      }
    }
  }
  sm[warp][0][lane] = m;
  sm[warp][1][lane] = s;
  sm[warp][2][lane] = u;
  sm[warp][3][lane] = q;
  __syncthreads();
  if (warp == 0 && r < rows) {
    for (int w = 1; w < 8; ++w) {
      m = fmaxf(m, sm[w][0][lane]);
      s += sm[w][1][lane];
      u += sm[w][2][lane];
      q += sm[w][3][lane];
    }
    const float ref = (row_ref_in != nullptr) ? row_ref_in[r] : 0.f;
    const long long yv = labels[r];
    const long long yl = yv - vocab_offset;
    const bool own = (yv != ignore_index) && yl >= 0 && yl < vocab_local;
    parts[0 * stat_ld + r] = ref;
    parts[1 * stat_ld + r] = s;
    parts[2 * stat_ld + r] = own ? target_logit[r] : 0.f;
    parts[3 * stat_ld + r] = u;
    parts[4 * stat_ld + r] = q;
    parts[5 * stat_ld + r] = m;
    row_base_out[r] = ref;
    row_ref_out[r] = m;
    if (!(m - ref <= kRefAbove && m - ref >= -kRefBelow)) {  // also catches NaN / inf
      *rescue = 1;
      rescue_groups[(group_row0 + r) >> 8] = 1;
    }
  }
}

// ref_i = max over the probed tiles of the tile maxima + kProbeMargin (see kProbeTiles).
__global__ void __launch_bounds__(256)
probe_ref_kernel(const float* __restrict__ tile_max, long long stat_ld, int tiles, int rows,
                 float* __restrict__ row_ref) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= rows) return;
  float m = -INFINITY;
  for (int t = 0; t < tiles; ++t) m = fmaxf(m, tile_max[(long long)t * stat_ld + r]);
  row_ref[r] = m + kProbeMargin;
}

// A value that another GPU may have stored while this kernel was already running (published through a flag that
// this kernel acquired): a plain coherent load, never the read-only path.
__device__ __forceinline__ float ld_coherent(const float* p) {
  float v;
  asm volatile("ld.global.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
  return v;
}

// Body of the combine step, for one block of 1024 threads per chunk. parts_all: [world][ROW_PARTS][stat_ld].
// rescue_groups: n_groups ints of this chunk's buffers; the last one is the chunk's "any group flagged" word.
template <bool kCoherent>
__device__ __forceinline__ void combine_rows(const float* parts_all, int world, const long long* __restrict__ labels,
                                             int rows, long long stat_ld, long long ignore_index, int monitoring,
                                             float* __restrict__ lse_out, PassScalars* sc, int* rescue_groups,
                                             int n_groups) {
  __shared__ double scratch_d[32];
  __shared__ float scratch_f[32];
  double a_nll = 0.0, a_lse2 = 0.0, a_ent = 0.0, a_norm = 0.0;
  float a_max = -INFINITY;
  auto get = [](const float* p) { return kCoherent ? ld_coherent(p) : __ldg(p); };
  for (int r = threadIdx.x; r < rows; r += blockDim.x) {
    float m = -INFINITY, s = 0.f, u = 0.f, t = 0.f, q = 0.f, zmax = -INFINITY;
    for (int g = 0; g < world; ++g) {
      const float* pg = parts_all + (long long)g * ROW_PARTS * stat_ld;
      lse_merge(m, s, u, get(pg + 0 * stat_ld + r), get(pg + 1 * stat_ld + r), get(pg + 3 * stat_ld + r));
      t += get(pg + 2 * stat_ld + r);
      q += get(pg + 4 * stat_ld + r);
      zmax = fmaxf(zmax, get(pg + 5 * stat_ld + r));
    }
    const float lse = m + logf(s);
    lse_out[r] = lse;
    const bool valid = labels[r] != ignore_index;
    if (valid) {
      a_nll += (double)lse - (double)t;
      a_lse2 += (double)lse * (double)lse;
      if (monitoring) a_ent += (double)lse - (double)u / (double)s;
    }
    if (monitoring) {
      a_norm += sqrt((double)q);
      a_max = fmaxf(a_max, zmax);
    }
  }
  const double t_nll = block_sum_double(a_nll, scratch_d);
  const double t_lse2 = block_sum_double(a_lse2, scratch_d);
  const double t_ent = block_sum_double(a_ent, scratch_d);
  const double t_norm = block_sum_double(a_norm, scratch_d);
  const float t_max = block_max_float(a_max, scratch_f);
  if (threadIdx.x == 0) {
    sc->sum_nll += t_nll;
    sc->sum_lse2 += t_lse2;
    sc->sum_ent += t_ent;
    sc->sum_norm += t_norm;
    sc->max_logit = fmaxf(sc->max_logit, t_max);
    int flagged = 0;
    for (int g = 0; g + 1 < n_groups; ++g) flagged += rescue_groups[g] != 0;
    sc->rerun_groups += flagged;
    sc->seen_groups += (rows + 255) >> 8;
  }
  __syncthreads();
  // the chunk's conditional re-run (if any) is behind us: clear its flags for the next chunk that uses these buffers
  for (int g = threadIdx.x; g < n_groups; g += blockDim.x) rescue_groups[g] = 0;
}

__global__ void __launch_bounds__(1024)
combine_kernel(const float* __restrict__ parts_all, int world, const long long* __restrict__ labels, int rows,
               long long stat_ld, long long ignore_index, int monitoring, float* __restrict__ lse_out,
               PassScalars* sc, int* rescue_groups, int n_groups) {
  combine_rows<false>(parts_all, world, labels, rows, stat_ld, ignore_index, monitoring, lse_out, sc, rescue_groups,
                      n_groups);
}

__global__ void finalize_kernel(const PassScalars* sc, double n_rows_total, float z_regularization,
                                float* __restrict__ out5) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  const double R = (double)sc->n_valid;
  double loss = (sc->sum_nll + (double)z_regularization * sc->sum_lse2) / R;  // R == 0 -> NaN, as in the reference
  if (sc->status != 0) loss = NAN;
  out5[0] = (float)loss;
  out5[1] = (float)(sc->sum_lse2 / R);
  out5[2] = sc->max_logit;
  out5[3] = (float)(sc->sum_ent / R);
  out5[4] = (float)(sc->sum_norm / n_rows_total);
}

// ---------------------------------------------------------------------------------------------
// slab transform: one warp per (row, V tile) segment of 256 elements, 8 elements per lane.
// ---------------------------------------------------------------------------------------------
template <typename T>
struct Vec8 {};
template <>
struct Vec8<__half> {
  uint4 raw;
  __device__ void load(const __half* p) { raw = *reinterpret_cast<const uint4*>(p); }
  __device__ void store(__half* p) const { *reinterpret_cast<uint4*>(p) = raw; }
  __device__ void to_float(float (&f)[8]) const {
    const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 v = __half22float2(h[i]);
      f[2 * i] = v.x;
      f[2 * i + 1] = v.y;
    }
  }
  __device__ void from_float(const float (&f)[8]) {
    __half2* h = reinterpret_cast<__half2*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
  }
};
template <>
struct Vec8<__nv_bfloat16> {
  uint4 raw;
  __device__ void load(const __nv_bfloat16* p) { raw = *reinterpret_cast<const uint4*>(p); }
  __device__ void store(__nv_bfloat16* p) const { *reinterpret_cast<uint4*>(p) = raw; }
  __device__ void to_float(float (&f)[8]) const {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 v = __bfloat1622float2(h[i]);
      f[2 * i] = v.x;
      f[2 * i + 1] = v.y;
    }
  }
  __device__ void from_float(const float (&f)[8]) {
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  }
};
template <>
struct Vec8<float> {
  float4 a, b;
  __device__ void load(const float* p) {
    a = *reinterpret_cast<const float4*>(p);
    b = *reinterpret_cast<const float4*>(p + 4);
  }
  __device__ void store(float* p) const {
    *reinterpret_cast<float4*>(p) = a;
    *reinterpret_cast<float4*>(p + 4) = b;
  }
  __device__ void to_float(float (&f)[8]) const {
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w;
    f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
  }
  __device__ void from_float(const float (&f)[8]) {
    a = make_float4(f[0], f[1], f[2], f[3]);
    b = make_float4(f[4], f[5], f[6], f[7]);
  }
};

// dZ[i, j] = valid_i * ( e[i, j] * exp(tile_max[i, tile(j)] - lse_i) * (1 + 2 z_reg lse_i) - [j == y_i] )
// rounded to the input element type, unscaled (logit_scale / n_valid is applied to the fp32
// accumulators of the two gradient GEMMs, as the reference does).
// Work item = (group of 8 rows, V tile); the 8 warps of a block take the 8 rows of the group.
template <typename T>
__global__ void __launch_bounds__(256)
dz_transform_kernel(T* __restrict__ slab, long long slab_ld, const float* __restrict__ tile_max,
                    const float* __restrict__ lse, const long long* __restrict__ labels, int rows, int rows_valid,
                    int n_tiles, long long stat_ld, long long ignore_index, long long vocab_offset,
                    float z_regularization) {
  // rows: multiple of 128 (slab rows to rewrite); rows >= rows_valid are padding and become zero
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long items = (long long)(rows / 8) * n_tiles;
  for (long long item = blockIdx.x; item < items; item += gridDim.x) {
    const int tile = (int)(item % n_tiles);
    const int r = (int)(item / n_tiles) * 8 + warp;
    const bool exists = r < rows_valid;
    const long long yv = exists ? labels[r] : ignore_index;
    const bool valid = (yv != ignore_index);
    const float lse_r = exists ? lse[r] : 0.f;
    const float coef =
        valid ? __expf(tile_max[(long long)tile * stat_ld + r] - lse_r) * (1.f + 2.f * z_regularization * lse_r)
              : 0.f;
    const long long ycol = yv - vocab_offset - (long long)tile * 256;
    T* ptr = slab + (long long)r * slab_ld + (long long)tile * 256 + lane * 8;
    Vec8<T> v;
    v.load(ptr);
    float f[8];
    v.to_float(f);
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] *= coef;
    if (valid && ycol >= 0 && ycol < 256 && (int)(ycol >> 3) == lane) {
      const int sel = (int)(ycol & 7);
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if (i == sel) f[i] -= 1.f;
    }
    v.from_float(f);
    v.store(ptr);
  }
}

// ---------------------------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ T cast_from_float(float v);
template <>
__device__ __forceinline__ float cast_from_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ __half cast_from_float<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 cast_from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

template <typename T>
__device__ __forceinline__ float cast_to_float(T v);
template <>
__device__ __forceinline__ float cast_to_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ float cast_to_float<__half>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float cast_to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

// Row-reference mode, after the log-sum-exp is known. One block per row:
//   C_i = valid_i * exp(ref_i - lse_i) * (1 + 2 z_reg lse_i)        -> row_coef[i]   (factor of dx), moved to the
//         nearest value whose reciprocal is a T number
//   xs[i, :] = C_i * x[i, :]                                        (A operand of dW = xs^T slab)
//   slab[i, y_i] -= 1 / C_i   if this rank owns column y_i          (so that C_i * slab[i, :] = dZ[i, :])
// ref_i is the base the row's partials were computed with (parts[0]).
template <typename T>
__global__ void __launch_bounds__(256)
row_finish_kernel(const T* __restrict__ x, long long x_ld, T* __restrict__ xs, long long xs_ld, int hidden,
                  T* __restrict__ slab, long long slab_ld, const float* __restrict__ ref, const float* __restrict__ lse,
                  const long long* __restrict__ labels, int rows_valid, long long ignore_index,
                  long long vocab_offset, long long vocab_local, float z_regularization,
                  float* __restrict__ row_coef) {
  // grid = rows rounded up to 128: blocks r >= rows_valid are padding rows (factor 0, zero xs row)
  const int r = blockIdx.x;
  const bool exists = r < rows_valid;
  const long long yv = exists ? labels[r] : ignore_index;
  const bool valid = (yv != ignore_index);
  const float l = exists ? lse[r] : 0.f;
  float C = valid ? __expf(ref[r] - l) * (1.f + 2.f * z_regularization * l) : 0.f;
  if (valid && fabsf(C) < 1e-30f) C = (C < 0.f) ? -1e-30f : 1e-30f;  // keeps 1 / C finite
  // The label entry carries the dominant term of the row's gradient (softmax - 1 is close to -1 there), so it is
  // kept exact: the factor is nudged (by at most half an ulp of T, the size of the rounding every softmax entry
  // gets anyway) to the nearest value whose reciprocal is representable in T. slab[i, y_i] - 1 / C then rounds
  // with an error relative to the softmax entry, not to 1 / C, and C * (that entry) is -1 + softmax to fp32 accuracy.
  float rcp = 0.f;
  if (valid) {
    rcp = cast_to_float<T>(cast_from_float<T>(1.f / C));
    C = 1.f / rcp;
  }
  if (threadIdx.x == 0) {
    row_coef[r] = C;
    const long long yl = yv - vocab_offset;
    if (valid && yl >= 0 && yl < vocab_local) {
      T* e = slab + (long long)r * slab_ld + yl;
      *e = cast_from_float<T>(cast_to_float<T>(*e) - rcp);
    }
  }
  const T* src = x + (long long)r * x_ld;
  T* dst = xs + (long long)r * xs_ld;
  for (int c = threadIdx.x * 8; c < hidden; c += blockDim.x * 8) {  // hidden % 8 == 0
    Vec8<T> v;
    float f[8];
    if (exists) {
      v.load(src + c);
      v.to_float(f);
#pragma unroll
      for (int k = 0; k < 8; ++k) f[k] *= C;
    } else {
#pragma unroll
      for (int k = 0; k < 8; ++k) f[k] = 0.f;
    }
    v.from_float(f);
    v.store(dst + c);
  }
}

// dx[r, h] = sum_s part[s][r][h]  (fixed order s = 0, 1, ...), cast to T. cols % 4 == 0.
template <typename T>
__global__ void __launch_bounds__(256)
dx_reduce_kernel(const float* __restrict__ part, int splits, long long split_stride, long long part_ld, int rows,
                 int cols, T* __restrict__ dx, long long dx_ld) {
  const long long quads = (long long)rows * (cols / 4);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < quads;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / (cols / 4);
    const int c = (int)(i % (cols / 4)) * 4;
    float4 acc = *reinterpret_cast<const float4*>(part + r * part_ld + c);
    for (int s = 1; s < splits; ++s) {
      const float4 v = *reinterpret_cast<const float4*>(part + (long long)s * split_stride + r * part_ld + c);
      acc.x += v.x;
      acc.y += v.y;
      acc.z += v.z;
      acc.w += v.w;
    }
    T* d = dx + r * dx_ld + c;
    d[0] = cast_from_float<T>(acc.x);
    d[1] = cast_from_float<T>(acc.y);
    d[2] = cast_from_float<T>(acc.z);
    d[3] = cast_from_float<T>(acc.w);
  }
}

// dst = src * (*factor) with a type conversion, 8 elements per thread (cols % 8 == 0, rows 16-byte aligned).
// When the call is an in-place rescale (skip_if_one) and the factor is exactly 1 nothing is touched: that is
// the usual loss.backward() case, where grad_output == 1.
template <typename S, typename D>
__global__ void __launch_bounds__(256)
scale_cast_kernel(const S* src, long long src_ld, D* dst, long long dst_ld, long long rows, long long cols,
                  const float* __restrict__ factor, int skip_if_one) {
  const float f = *factor;
  if (skip_if_one && f == 1.0f) return;
  const long long per_row = cols / 8;
  const long long n = rows * per_row;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / per_row, c = (i - r * per_row) * 8;
    Vec8<S> in;
    in.load(src + r * src_ld + c);
    float v[8];
    in.to_float(v);
#pragma unroll
    for (int k = 0; k < 8; ++k) v[k] *= f;
    Vec8<D> out;
    out.from_float(v);
    out.store(dst + r * dst_ld + c);
  }
}

}  // namespace lce
