// Multi-tensor-apply plumbing shared by every optimizer kernel (sm_100a).
//
// One launch covers a whole list of tensors.  The list is described by an MtaTable passed BY VALUE
// in kernel parameter space (up to ~30 KB, which sm_70+ devices accept since CUDA 12.1), so a step
// needs no device-side metadata buffer, no host-to-device copy and no allocation.  Tensors are cut
// into fixed-size chunks; block b handles chunk b and finds its tensor with a binary search over
// the prefix sum of chunk counts.  Within a chunk every thread moves 16 bytes per stream per
// iteration (8 x bf16/fp16 or 4 x fp32), fully coalesced, with streaming cache hints since each
// byte is touched once per step.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace optimi {

constexpr int kThreads = 512;          // threads per block
constexpr int kTableBytes = 30720;     // budget for one by-value table
constexpr int kMinChunk = 4096;        // elements; multiple of kThreads * 8
constexpr int kMaxChunk = 65536;

template <int NL>
struct MtaTable {
  static constexpr int CAP = kTableBytes / (NL * 8 + 12);
  void* ptr[NL][CAP];        // ptr[list][tensor]
  long long numel[CAP];
  int chunk_start[CAP + 1];  // prefix sum of chunks per tensor; chunk_start[n_tensors] = grid size
  int n_tensors;
  int chunk_elems;
  int tensor_base;           // index of tensor 0 of this table within the caller's whole list
  int chunk_base;            // index of chunk 0 of this table within the caller's whole list
};

// ---------------------------------------------------------------------------------------------
// rounding to the storage type (round to nearest even), returned as float
// ---------------------------------------------------------------------------------------------
template <typename T> __device__ __forceinline__ float rnd(float x);
template <> __device__ __forceinline__ float rnd<float>(float x) { return x; }
template <> __device__ __forceinline__ float rnd<__nv_bfloat16>(float x) {
  return __bfloat162float(__float2bfloat16_rn(x));
}
template <> __device__ __forceinline__ float rnd<__half>(float x) { return __half2float(__float2half_rn(x)); }

// ---------------------------------------------------------------------------------------------
// 16-byte vector access.  N = elements per vector.
// ---------------------------------------------------------------------------------------------
template <typename T> struct VecN;
template <> struct VecN<float> { static constexpr int N = 4; };
template <> struct VecN<__nv_bfloat16> { static constexpr int N = 8; };
template <> struct VecN<__half> { static constexpr int N = 8; };

__device__ __forceinline__ uint4 ld_stream(const void* p) { return __ldcs(reinterpret_cast<const uint4*>(p)); }
__device__ __forceinline__ void st_stream(void* p, uint4 v) { __stcs(reinterpret_cast<uint4*>(p), v); }

template <typename T, int N> struct Pack;

// full vector
template <> struct Pack<float, 4> {
  static __device__ __forceinline__ void load(const float* p, float (&x)[4]) {
    uint4 r = ld_stream(p);
    x[0] = __uint_as_float(r.x); x[1] = __uint_as_float(r.y); x[2] = __uint_as_float(r.z); x[3] = __uint_as_float(r.w);
  }
  static __device__ __forceinline__ void store(float* p, const float (&x)[4]) {
    st_stream(p, make_uint4(__float_as_uint(x[0]), __float_as_uint(x[1]), __float_as_uint(x[2]), __float_as_uint(x[3])));
  }
};
template <> struct Pack<__nv_bfloat16, 8> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&x)[8]) {
    uint4 r = ld_stream(p);
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {  // bf16 -> fp32 is a 16-bit shift
      x[2 * i] = __uint_as_float(w[i] << 16);
      x[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&x)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
      __nv_bfloat162 h = __floats2bfloat162_rn(x[2 * i], x[2 * i + 1]);
      w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    st_stream(p, make_uint4(w[0], w[1], w[2], w[3]));
  }
};
template <> struct Pack<__half, 8> {
  static __device__ __forceinline__ void load(const __half* p, float (&x)[8]) {
    uint4 r = ld_stream(p);
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
      float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
      x[2 * i] = f.x; x[2 * i + 1] = f.y;
    }
  }
  static __device__ __forceinline__ void store(__half* p, const float (&x)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
      __half2 h = __floats2half2_rn(x[2 * i], x[2 * i + 1]);
      w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    st_stream(p, make_uint4(w[0], w[1], w[2], w[3]));
  }
};
// single element (ragged tails, tensors whose base address is not 16-byte aligned)
template <> struct Pack<float, 1> {
  static __device__ __forceinline__ void load(const float* p, float (&x)[1]) { x[0] = *p; }
  static __device__ __forceinline__ void store(float* p, const float (&x)[1]) { *p = x[0]; }
};
template <> struct Pack<__nv_bfloat16, 1> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&x)[1]) { x[0] = __bfloat162float(*p); }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&x)[1]) { *p = __float2bfloat16_rn(x[0]); }
};
template <> struct Pack<__half, 1> {
  static __device__ __forceinline__ void load(const __half* p, float (&x)[1]) { x[0] = __half2float(*p); }
  static __device__ __forceinline__ void store(__half* p, const float (&x)[1]) { *p = __float2half_rn(x[0]); }
};

// ---------------------------------------------------------------------------------------------
// fp32 building blocks with the exact formula of the ATen CUDA op they replay
// ---------------------------------------------------------------------------------------------
// at::native::lerp with a scalar weight: |w| < 0.5 ? a + w*(b-a) : b - (b-a)*(1-w), multiply and
// add fused.  `low` = (|w| < 0.5), `omw` = 1 - w, both uniform across the launch.
__device__ __forceinline__ float lerp_op(float a, float b, float w, float omw, bool low) {
  float d = __fsub_rn(b, a);
  return low ? __fmaf_rn(w, d, a) : __fmaf_rn(-d, omw, b);
}

// ---------------------------------------------------------------------------------------------
// chunk location
// ---------------------------------------------------------------------------------------------
struct Span {
  int tensor;         // index within the table
  long long begin;    // first element of this block's chunk within the tensor
  int len;            // elements in this chunk (<= chunk_elems)
};

template <int NL>
__device__ __forceinline__ Span locate(const MtaTable<NL>& tab, int chunk) {
  int lo = 0, hi = tab.n_tensors;  // invariant: chunk_start[lo] <= chunk < chunk_start[hi]
  while (hi - lo > 1) {
    int mid = (lo + hi) >> 1;
    if (tab.chunk_start[mid] <= chunk) lo = mid; else hi = mid;
  }
  Span s;
  s.tensor = lo;
  s.begin = (long long)(chunk - tab.chunk_start[lo]) * tab.chunk_elems;
  long long rem = tab.numel[lo] - s.begin;
  s.len = rem < tab.chunk_elems ? (int)rem : tab.chunk_elems;
  return s;
}

// Fetches the block's base pointers (advanced to the chunk) and reports whether every present
// list is 16-byte aligned there; chunk offsets are multiples of 4096 elements, so only the
// tensors' base addresses decide.
template <typename T, int NL>
__device__ __forceinline__ bool chunk_pointers(const MtaTable<NL>& tab, const Span& s, T* (&p)[NL]) {
  uintptr_t bits = 0;
#pragma unroll
  for (int l = 0; l < NL; l++) {
    T* base = reinterpret_cast<T*>(tab.ptr[l][s.tensor]);
    bits |= reinterpret_cast<uintptr_t>(base);
    p[l] = base ? base + s.begin : nullptr;
  }
  return (bits & 15) == 0;
}

// Generic element-wise kernel: Op::run<T, N>(pointers, element offset, args) handles N consecutive
// elements (N = vector width or 1).
template <typename T, class Op>
__global__ void __launch_bounds__(kThreads) mta_kernel(const __grid_constant__ MtaTable<Op::NL> tab,
                                                       const __grid_constant__ typename Op::Args args) {
  constexpr int V = VecN<T>::N;
  const Span s = locate(tab, blockIdx.x);
  T* p[Op::NL];
  const bool aligned = chunk_pointers<T, Op::NL>(tab, s, p);
  if (aligned) {
    const int nvec = s.len / V;
#pragma unroll 2
    for (int i = threadIdx.x; i < nvec; i += kThreads) Op::template run<T, V>(p, i * V, args);
    for (int i = nvec * V + threadIdx.x; i < s.len; i += kThreads) Op::template run<T, 1>(p, i, args);
  } else {
    for (int i = threadIdx.x; i < s.len; i += kThreads) Op::template run<T, 1>(p, i, args);
  }
}

}  // namespace optimi
