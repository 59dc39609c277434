// Exchange of the dx partials between the GPUs of a vocabulary-sharded run, over peer-mapped memory.
//
// Every rank holds one exchange buffer that all ranks of the node can address (NVLink / NVSwitch peer
// mapping; the caller allocates it and passes the table of base addresses). Layout of one buffer:
//
//   [ flags: 2 phases x 8 senders, uint32 ]  (padded to 1 KiB)
//   [ recv[2] : fp32 [slots][rows_own][h_pad] ]   slots = world * splits, rows_own = chunk_rows / world
//   [ stage[2]: dx dtype [chunk_rows][hidden] ]
//
// One chunk's dx then takes three steps, all of them plain stream-ordered launches:
//   1. the dx contraction stores every fp32 output tile straight into the recv buffer of the rank that
//      owns those rows (its epilogue is the sender: the transfer runs tile by tile under the math), then
//      a one-warp kernel publishes flag A = epoch to every rank;
//   2. the owner waits for flag A of every sender, sums the slots in a fixed order (rank-major, then
//      split), rounds once to the dx dtype and stores the rows into the stage buffer of every rank;
//      a one-warp kernel publishes flag B;
//   3. every rank waits for flag B of every owner and copies the staged rows into its dx tensor.
// Only stores and flags cross the links; all loads are local. Each row is summed by exactly one rank and
// broadcast, so dx is bitwise identical on all ranks and independent of timing.
//
// recv/stage are double-buffered by epoch parity so that step 2/3 of one chunk may run on a second
// stream underneath the next contractions. Epochs grow by one per chunk over the life of the buffer;
// flags are compared as signed differences.
//
// Every wait is bounded by wall time (globaltimer): on expiry the kernel records DEV_WAIT_TIMEOUT_PEER in
// the status word and returns without touching data; the loss of that pass becomes NaN.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace lce {

constexpr int kMaxPeers = 8;
constexpr size_t kPeerFlagBytes = 1024;
enum : int { DEV_WAIT_TIMEOUT_PEER = 104 };

struct PeerBases {
  unsigned char* base[kMaxPeers];
};

struct PeerLayout {
  int slots;           // world * splits
  int rows_own;        // chunk_rows / world
  size_t recv_bytes;   // one recv buffer
  size_t stage_bytes;  // one stage buffer
  size_t total;
  __host__ __device__ size_t recv_off(int buf) const { return kPeerFlagBytes + size_t(buf) * recv_bytes; }
  __host__ __device__ size_t stage_off(int buf) const {
    return kPeerFlagBytes + 2 * recv_bytes + size_t(buf) * stage_bytes;
  }
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float4 ld_global_f4(const float* p) {
  float4 v;
  asm volatile("ld.global.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long wall_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// flag[phase][rank] = epoch in every rank's buffer. Launched after the kernel whose stores it publishes:
// the kernel boundary orders those stores before this thread, the system-scope fence and release before
// the flag.
// skip_if: when non-null and *skip_if != 0 (the pass's status word after a wait of the preceding kernel ran
// out, so that kernel wrote nothing) the flag is NOT published: the other ranks' waits then run out too and
// they report the failure instead of copying rows that were never written.
__global__ void peer_signal_kernel(PeerBases peers, int world, int rank, int phase, uint32_t epoch,
                                   const int* skip_if) {
  const int t = threadIdx.x;
  if (skip_if != nullptr && *skip_if != 0) return;
  if (t < world) {
    __threadfence_system();
    st_release_sys(reinterpret_cast<uint32_t*>(peers.base[t]) + phase * kMaxPeers + rank, epoch);
  }
}

// All threads of the CTA call this. Threads 0..world-1 poll one sender's flag each until it has reached
// `epoch` or `limit_ns` has passed; returns true for the whole CTA iff every flag arrived.
__device__ __forceinline__ bool peer_wait_all(const uint32_t* flags, int world, uint32_t epoch, long long limit_ns,
                                              int* status) {
  __shared__ int s_fail;
  // A pass whose status word is already set (an earlier wait of this pass ran out) does not wait again: its loss is
  // NaN whatever follows, and one expired wait per pass bounds the time a broken exchange can cost.
  if (threadIdx.x == 0) s_fail = (*reinterpret_cast<volatile int*>(status) != 0) ? 1 : 0;
  __syncthreads();
  if (s_fail == 0 && threadIdx.x < world) {
    const unsigned long long t0 = wall_ns();
    while (int32_t(ld_acquire_sys(flags + threadIdx.x) - epoch) < 0) {
      if ((long long)(wall_ns() - t0) > limit_ns) {
        s_fail = 1;
        atomicCAS(status, 0, DEV_WAIT_TIMEOUT_PEER);
        break;
      }
      __nanosleep(500);
    }
  }
  __syncthreads();
  return s_fail == 0;
}

// ---------------------------------------------------------------------------------------------
// Exchange of the per-row softmax partials (replaces an all-gather). Buffer of one rank:
//   [ flags: 8 senders, uint32 ] (padded to 1 KiB)   [ 4 slots x [world][ROW_PARTS][chunk_rows] fp32 ]
// A sender copies its [ROW_PARTS][rows] block into slot (epoch % 4), position `rank`, of EVERY rank's buffer
// (parts_push_kernel), then peer_signal_kernel publishes flag[rank] = epoch everywhere. The combine step of a rank
// waits for all flags to reach the epoch and merges the blocks in rank order.
// ---------------------------------------------------------------------------------------------
constexpr int kPartsSlots = 4;
__host__ __device__ inline size_t parts_slot_bytes(int world, long long chunk_rows) {
  return (size_t(world) * ROW_PARTS * size_t(chunk_rows) * sizeof(float) + 255) / 256 * 256;
}
__host__ __device__ inline size_t parts_slot_off(int world, long long chunk_rows, uint32_t epoch) {
  return kPeerFlagBytes + size_t(epoch % kPartsSlots) * parts_slot_bytes(world, chunk_rows);
}

// local: [ROW_PARTS][stat_ld] of this rank; rows [row_lo, row_lo + rows) of each of the ROW_PARTS arrays are sent.
__global__ void __launch_bounds__(256)
parts_push_kernel(PeerBases peers, int world, int rank, const float* __restrict__ local, long long stat_ld, int row_lo,
                  int rows, size_t slot_off) {
  const long long per_peer = (long long)ROW_PARTS * rows;
  const long long total = per_peer * world;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int g = int(i / per_peer);
    const long long j = i - (long long)g * per_peer;
    const int q = int(j / rows);
    const int r = row_lo + int(j - (long long)q * rows);
    float* dst = reinterpret_cast<float*>(peers.base[g] + slot_off) + ((long long)rank * ROW_PARTS + q) * stat_ld + r;
    *dst = local[(long long)q * stat_ld + r];
  }
}

// lce_combine_chunk for a sharded run whose partials arrive through the exchange buffer: one block; waits for the
// flags of all ranks first. On expiry nothing is merged and the status word makes the loss of the pass NaN.
__global__ void __launch_bounds__(1024)
combine_peer_kernel(const uint32_t* flags, uint32_t epoch, long long limit_ns, const float* parts_all, int world,
                    const long long* __restrict__ labels, int rows, long long stat_ld, long long ignore_index,
                    int monitoring, float* __restrict__ lse_out, PassScalars* sc, int* rescue_groups, int n_groups) {
  if (!peer_wait_all(flags, world, epoch, limit_ns, &sc->status)) return;
  combine_rows<true>(parts_all, world, labels, rows, stat_ld, ignore_index, monitoring, lse_out, sc, rescue_groups,
                     n_groups);
}

template <typename T>
struct Pack8;
template <>
struct Pack8<float> {
  static __device__ __forceinline__ void store(float* dst, const float (&v)[8]) {
    reinterpret_cast<float4*>(dst)[0] = make_float4(v[0], v[1], v[2], v[3]);
    reinterpret_cast<float4*>(dst)[1] = make_float4(v[4], v[5], v[6], v[7]);
  }
};
template <>
struct Pack8<__half> {
  static __device__ __forceinline__ void store(__half* dst, const float (&v)[8]) {
    __half2 h[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<uint4*>(h);
  }
};
template <>
struct Pack8<__nv_bfloat16> {
  static __device__ __forceinline__ void store(__nv_bfloat16* dst, const float (&v)[8]) {
    __nv_bfloat162 h[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<uint4*>(h);
  }
};

// Step 2: sum the slots of the rows this rank owns and store the result into every rank's stage buffer.
// recv: this rank's receive buffer [slots][rows_own][ld]; rows [own_lo, own_hi) of it exist in this chunk
// (indices local to the owned slice); chunk_row0 = chunk-local index of owned row 0.
template <typename T>
__global__ void peer_reduce_push_kernel(PeerBases peers, int world, const uint32_t* flags_a, uint32_t epoch,
                                        long long limit_ns, const float* recv, int slots, int rows_own,
                                        int ld, int own_lo, int own_hi, int chunk_row0, int hidden,
                                        size_t stage_off, int* status) {
  if (!peer_wait_all(flags_a, world, epoch, limit_ns, status)) return;
  const int octs = hidden >> 3;
  const long long total = (long long)(own_hi - own_lo) * octs;
  const size_t slot_stride = size_t(rows_own) * ld;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int r = own_lo + int(i / octs);
    const int c = int(i % octs) << 3;
    const float* src = recv + size_t(r) * ld + c;
    float acc[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[k] = 0.f;
    for (int s = 0; s < slots; ++s) {
      // recv was written by other GPUs while this kernel may already have been running: plain coherent loads
      // (never the read-only path, which is only defined for data that no one writes during the kernel)
      const float4 a = ld_global_f4(src + s * slot_stride);
      const float4 b = ld_global_f4(src + s * slot_stride + 4);
      acc[0] += a.x, acc[1] += a.y, acc[2] += a.z, acc[3] += a.w;
      acc[4] += b.x, acc[5] += b.y, acc[6] += b.z, acc[7] += b.w;
    }
    const size_t elem = size_t(chunk_row0 + r) * hidden + c;
    for (int g = 0; g < world; ++g) Pack8<T>::store(reinterpret_cast<T*>(peers.base[g] + stage_off) + elem, acc);
  }
}

// Step 3: copy rows [row_lo, row_lo + rows) (chunk-local) of this rank's stage buffer into dx.
template <typename T>
__global__ void peer_finish_kernel(const uint32_t* flags_b, int world, uint32_t epoch, long long limit_ns,
                                   const T* stage, int row_lo, int rows, int hidden, T* __restrict__ dx_rows,
                                   long long dx_ld, int* status) {
  if (!peer_wait_all(flags_b, world, epoch, limit_ns, status)) return;
  const int octs = hidden >> 3;
  const long long total = (long long)rows * octs;
  constexpr int kVec = 16 / sizeof(T);  // elements per 16-byte access
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int r = int(i / octs);
    const int c = int(i % octs) << 3;
    const T* src = stage + size_t(row_lo + r) * hidden + c;
    T* dst = dx_rows + (long long)r * dx_ld + c;
#pragma unroll
    for (int v = 0; v < 8 / kVec; ++v)
      reinterpret_cast<float4*>(dst)[v] = ld_global_f4(reinterpret_cast<const float*>(src) + 4 * v);
  }
}

}  // namespace lce
