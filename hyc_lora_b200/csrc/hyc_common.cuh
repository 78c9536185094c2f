// Shared device helpers for the row-streaming kernels (sm_100a).
//
// Every kernel in this library walks rows of an activation.  A CTA owns a set
// of rows (row = blockIdx.x + i*gridDim.x), stages each row -- and whatever
// else the row needs (gradient row, packed codes) -- in shared memory with 1-D
// bulk asynchronous copies (cp.async.bulk, completion on an mbarrier), several
// stages deep, and makes a few cheap passes over the staged data.  No kernel
// waits on another CTA; the only waits are on a CTA's own copies and they are
// bounded.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

namespace hyc {

// Kernels this library has launched in this process (host-side bookkeeping, read through
// hyc_launch_count(); a benchmark uses the difference across its timed region).
extern std::atomic<unsigned long long> g_launch_count;
#define HYC_LAUNCHED() ((void)::hyc::g_launch_count.fetch_add(1ull, std::memory_order_relaxed))

constexpr int kMaxStages = 4;
constexpr uint32_t kStatusPoolOverflow = 1u;
constexpr uint32_t kStatusWaitExpired = 2u;

// ---------------------------------------------------------------- PTX wrappers

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

// make the initialised barriers visible to the asynchronous proxy
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

// order this thread's generic-proxy shared-memory accesses before later
// asynchronous-proxy (bulk copy) accesses to the same locations
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}

// 1-D bulk copy global -> this CTA's shared memory; both addresses 16-byte
// aligned, bytes a multiple of 16.  No multicast.
__device__ __forceinline__ void bulk_g2s(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          smem_u32(dst_smem)),
      "l"(__cvta_generic_to_global(src_gmem)), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait: gives up after `limit` SM clocks (by default about a second) and reports false.
constexpr long long kWaitCycles = 2000000000LL;
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, long long limit = kWaitCycles) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long start = clock64();
  while (!mbar_try_wait(bar, parity)) {
    if (clock64() - start > limit) return false;
  }
  return true;
}

// ---------------------------------------------------------------- bf16 helpers

__device__ __forceinline__ float bf16_bits_to_float(uint32_t bits16) { return __uint_as_float(bits16 << 16); }

// round-to-nearest-even to bf16, returned as fp32
__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

__device__ __forceinline__ uint32_t float_to_bf16_bits(float x) {
  return static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(x)));
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ void unpack_bf16x8(const uint4& w, float (&f)[8]) {
  f[0] = __uint_as_float(w.x << 16);
  f[1] = __uint_as_float(w.x & 0xffff0000u);
  f[2] = __uint_as_float(w.y << 16);
  f[3] = __uint_as_float(w.y & 0xffff0000u);
  f[4] = __uint_as_float(w.z << 16);
  f[5] = __uint_as_float(w.z & 0xffff0000u);
  f[6] = __uint_as_float(w.w << 16);
  f[7] = __uint_as_float(w.w & 0xffff0000u);
}

__device__ __forceinline__ uint4 pack_bf16x8(const float (&f)[8]) {
  uint4 w;
  w.x = pack_bf16x2(f[0], f[1]);
  w.y = pack_bf16x2(f[2], f[3]);
  w.z = pack_bf16x2(f[4], f[5]);
  w.w = pack_bf16x2(f[6], f[7]);
  return w;
}

// Load 8 consecutive elements (column `col`, multiple of 8) of a row as fp32.
// Works for shared or global rows (generic addressing), 16-byte aligned.
template <typename T>
__device__ __forceinline__ void load8(const T* row, int col, float (&f)[8]);

template <>
__device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* row, int col, float (&f)[8]) {
  const uint4 w = *reinterpret_cast<const uint4*>(row + col);
  unpack_bf16x8(w, f);
}

template <>
__device__ __forceinline__ void load8<float>(const float* row, int col, float (&f)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(row + col);
  const float4 b = *reinterpret_cast<const float4*>(row + col + 4);
  f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w;
  f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}

// fp32 tables of D entries that every thread reads 8 consecutive channels at a time (norm weights,
// reciprocal scales) are kept in shared memory with the two halves of each group of 8 apart:
// channel c sits at ((c >> 2) & 1) * D/2 + (c >> 3) * 4 + (c & 3).  A warp's two 16-byte reads
// then touch consecutive 16-byte pieces instead of every other one: no bank conflicts.
__device__ __forceinline__ int split_index(int c, int D) { return ((c >> 2) & 1) * (D >> 1) + ((c >> 3) << 2) + (c & 3); }
__device__ __forceinline__ void load8_split(const float* table, int D, int col, float (&f)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(table + ((col >> 3) << 2));
  const float4 b = *reinterpret_cast<const float4*>(table + (D >> 1) + ((col >> 3) << 2));
  f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w;
  f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}

template <typename T>
__device__ __forceinline__ void store8(T* row, int col, const float (&f)[8]);

template <>
__device__ __forceinline__ void store8<__nv_bfloat16>(__nv_bfloat16* row, int col, const float (&f)[8]) {
  *reinterpret_cast<uint4*>(row + col) = pack_bf16x8(f);
}

template <>
__device__ __forceinline__ void store8<float>(float* row, int col, const float (&f)[8]) {
  *reinterpret_cast<float4*>(row + col) = make_float4(f[0], f[1], f[2], f[3]);
  *reinterpret_cast<float4*>(row + col + 4) = make_float4(f[4], f[5], f[6], f[7]);
}

// ---------------------------------------------------------------- packed fp32 pairs

// Two fp32 values in one 64-bit register pair, for the packed fp32 instructions of sm_100
// (add / sub / mul / fma .f32x2: two IEEE operations, round to nearest even, per issue slot).
typedef unsigned long long f32x2;
__device__ __forceinline__ f32x2 f2_make(float lo, float hi) {
  f32x2 d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "f"(lo), "f"(hi));
  return d;
}
__device__ __forceinline__ void f2_split(f32x2 v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ f32x2 f2_add(f32x2 a, f32x2 b) {
  f32x2 d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ f32x2 f2_sub(f32x2 a, f32x2 b) {
  f32x2 d;
  asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ f32x2 f2_mul(f32x2 a, f32x2 b) {
  f32x2 d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ f32x2 f2_fma(f32x2 a, f32x2 b, f32x2 c) {
  f32x2 d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
// the eight bf16 values of a 16-byte piece as four fp32 pairs
__device__ __forceinline__ void unpack_bf16x8_pairs(const uint4& w, f32x2 (&f)[4]) {
  f[0] = f2_make(__uint_as_float(w.x << 16), __uint_as_float(w.x & 0xffff0000u));
  f[1] = f2_make(__uint_as_float(w.y << 16), __uint_as_float(w.y & 0xffff0000u));
  f[2] = f2_make(__uint_as_float(w.z << 16), __uint_as_float(w.z & 0xffff0000u));
  f[3] = f2_make(__uint_as_float(w.w << 16), __uint_as_float(w.w & 0xffff0000u));
}

// ---------------------------------------------------------------- reductions

struct OpSum {
  __device__ __forceinline__ float operator()(float a, float b) const { return a + b; }
};
struct OpMax {
  __device__ __forceinline__ float operator()(float a, float b) const { return fmaxf(a, b); }
};

// CTA-wide reduction of N values; every thread gets the result.  `slot` is a
// private shared array of N*32 floats for this call site; the same slot may be
// reused once per row because at least one __syncthreads separates the uses.
template <int N, class Op>
__device__ __forceinline__ void block_reduce(float (&v)[N], float* slot, Op op) {
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int nwarps = blockDim.x >> 5;
#pragma unroll
  for (int i = 0; i < N; ++i) {
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) v[i] = op(v[i], __shfl_xor_sync(0xffffffffu, v[i], m));
  }
  if (nwarps == 1) return;
  if (lane == 0) {
#pragma unroll
    for (int i = 0; i < N; ++i) slot[i * 32 + warp] = v[i];
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < N; ++i) {
    float r = slot[i * 32];
    for (int w = 1; w < nwarps; ++w) r = op(r, slot[i * 32 + w]);
    v[i] = r;
  }
}

// ---------------------------------------------------------------- staged rows

// Shared-memory ring of `stages` slots, one mbarrier per slot.  Thread 0 issues
// the copies of a row into a slot; everybody waits on the slot's barrier.
struct RowRing {
  uint64_t* bars;        // [stages]
  unsigned char* slots;  // stages * slot_bytes, 128-byte aligned
  uint32_t slot_bytes;
  int stages;
  long long wait_cycles = kWaitCycles;   // limit of every wait on this ring's barriers

  __device__ __forceinline__ unsigned char* slot(int s) const { return slots + static_cast<size_t>(s) * slot_bytes; }

  __device__ __forceinline__ void init() {
    if (threadIdx.x == 0) {
      for (int s = 0; s < stages; ++s) mbar_init(&bars[s], 1);
      fence_barrier_init();
    }
    __syncthreads();
  }
};

}  // namespace hyc
