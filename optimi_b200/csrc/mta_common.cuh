// Multi-tensor-apply plumbing shared by every optimizer kernel (sm_100a).
//
// One launch covers a whole list of tensors.  The list is described by an MtaTable passed BY VALUE
// in kernel parameter space (up to ~30 KB, which sm_70+ devices accept since CUDA 12.1), so a step
// needs no device-side metadata buffer, no host-to-device copy and no allocation.
//
// Work decomposition, chosen by measurement on a B200: tensors are cut into small fixed tiles of
// kThreads * U vectors (16 bytes each); one 128-thread block owns one tile, issues ALL of its loads
// up front (U vectors per stream per thread), computes, stores and exits.  Millions of short-lived
// blocks keep every SM's memory pipeline full without a persistent loop, and a register budget
// of 40 leaves twelve blocks resident per SM.  Block b finds its tensor through a 256-entry
// coarse index over the block range plus a short forward walk over the prefix sum of block counts
// (a plain binary search over the table cost 10-20 % of the step: every probe is a dependent,
// dynamically indexed read of kernel-parameter space).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace optimi {

constexpr int kThreads = 128;       // threads per block
constexpr int kTableBytes = 29440;  // budget for the per-tensor arrays of one by-value table
constexpr int kBuckets = 256;       // coarse index over the tile range (see locate)

// SMALL = true is the few-tensor form (gradient release steps one parameter per launch): a table of a
// few hundred bytes instead of ~30 KB keeps the launch itself cheap.
template <int NL, bool SMALL = false>
struct MtaTable {
  static constexpr int CAP = SMALL ? 4 : kTableBytes / (NL * 8 + 12);
  static constexpr int NB = SMALL ? 4 : kBuckets;
  void* ptr[NL][CAP];       // ptr[list][tensor]
  long long numel[CAP];
  int tile_start[CAP + 1];  // prefix sum of blocks per tensor; tile_start[n_tensors] = grid size
  // bucket_tensor[b] = tensor that owns block (b << bucket_shift): a block starts its search there
  // and walks forward, which for lists of large tensors is zero or one step
  int bucket_tensor[NB];
  int bucket_shift;
  int n_tensors;
  int tensor_base;          // index of tensor 0 of this table within the caller's whole list
  int tile_base;            // index of tile 0 of this table within the caller's whole list
};

// ---------------------------------------------------------------------------------------------
// storage types.  VecN<T>::N = elements per 16-byte vector.
// ---------------------------------------------------------------------------------------------
template <typename T> struct VecN;
template <> struct VecN<float> { static constexpr int N = 4; };
template <> struct VecN<__nv_bfloat16> { static constexpr int N = 8; };
template <> struct VecN<__half> { static constexpr int N = 8; };

// Round an fp32 value to the storage type (nearest even) and return it as fp32.
template <typename T> __device__ __forceinline__ float rnd(float x);
template <> __device__ __forceinline__ float rnd<float>(float x) { return x; }
template <> __device__ __forceinline__ float rnd<__nv_bfloat16>(float x) {
  // one instruction: convert the pair {x, 0} to packed bf16x2; x lands in the upper half, which is
  // exactly the fp32 bit pattern of the rounded value
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(x), "f"(0.0f));
  return __uint_as_float(r);
}
template <> __device__ __forceinline__ float rnd<__half>(float x) { return __half2float(__float2half_rn(x)); }

// sqrt followed by rounding to the storage type.  For bf16 inputs the approximate square root
// (relative error below 2^-22) rounds to the same bf16 value as the correctly rounded one: the
// square root of a number with an 8-bit significand stays at least 2^-18 (relative) away from every
// midpoint between two bf16 values.  fp16 and fp32 use the IEEE square root.
template <typename T> __device__ __forceinline__ float sqrt_rnd(float x) { return rnd<T>(__fsqrt_rn(x)); }
template <> __device__ __forceinline__ float sqrt_rnd<__nv_bfloat16>(float x) {
  float r;
  asm("sqrt.approx.f32 %0, %1;" : "=f"(r) : "f"(x));
  return rnd<__nv_bfloat16>(r);
}

// Correctly rounded fp32 quotient a / b of two values of a 16-bit storage type, given y = rcp_fast(b):
// one residual correction on an approximate reciprocal.  A quotient of two significands of at most
// 11 bits is either exactly representable in fp32 or at least 2^-36 (relative) away from every fp32
// rounding boundary, and q = q0 + (a - b*q0)*y is within 2^-44 of a/b, so q IS the rounded quotient —
// provided the residual does not underflow and the quotient is a normal number (|a| >= 2^-60 suffices,
// b being at most 2^65 as a square root plus eps) and nothing overflowed on the way.  Every failure of
// the second kind (b zero, subnormal, infinite or NaN, a infinite or NaN, a*y out of range) turns q
// into a NaN, so one test of |a| and one of q guard the shortcut.  What they turn away is rare and goes
// one of two ways: a zero numerator is answered by q0 = a*y itself (a zero of the right sign for any
// finite positive b, a NaN for b = 0, as the IEEE quotient), everything else by the IEEE division, kept
// out of line so that the common path does not carry its instruction sequence along.  Checked on the
// host against the double-precision quotient for all pairs of 8-bit significands with a in
// 2^-60..2^127, b in 2^-126..2^65, and all pairs of 11-bit significands over the float16 range, with
// the reciprocal off by -2..+2 units: no wrong result passes the guard.
__device__ __forceinline__ float rcp_fast(float b) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(b));
  return y;
}
static __device__ __noinline__ float div_ieee(float a, float b) { return __fdiv_rn(a, b); }
__device__ __forceinline__ float div16(float a, float b, float y) {
  const float q0 = __fmul_rn(a, y);
  const float r = __fmaf_rn(-b, q0, a);
  float q = __fmaf_rn(r, y, q0);
  if (__builtin_expect(!(fabsf(a) >= 0x1p-60f) || q != q, 0)) q = a == 0.f ? q0 : div_ieee(a, b);
  return q;
}

// Unpack a 16-byte vector into fp32 (exact) and pack fp32 values that are already representable in T.
template <typename T> struct Pack;
template <> struct Pack<float> {
  static constexpr int EPW = 1;  // elements per 32-bit word
  static __device__ __forceinline__ void unpack_word(uint32_t w, float (&x)[1]) { x[0] = __uint_as_float(w); }
  static __device__ __forceinline__ uint32_t pack_word(const float (&x)[1]) { return __float_as_uint(x[0]); }
  static __device__ __forceinline__ void unpack(uint4 r, float (&x)[4]) {
    x[0] = __uint_as_float(r.x); x[1] = __uint_as_float(r.y); x[2] = __uint_as_float(r.z); x[3] = __uint_as_float(r.w);
  }
  static __device__ __forceinline__ uint4 pack(const float (&x)[4]) {
    return make_uint4(__float_as_uint(x[0]), __float_as_uint(x[1]), __float_as_uint(x[2]), __float_as_uint(x[3]));
  }
  static __device__ __forceinline__ float load1(const float* p) { return *p; }
  static __device__ __forceinline__ void store1(float* p, float x) { *p = x; }
  static __device__ __forceinline__ void kahan2(uint32_t&, uint32_t&) {}  // no Kahan compensation in fp32 storage
};
template <> struct Pack<__nv_bfloat16> {
  static constexpr int EPW = 2;
  static __device__ __forceinline__ void unpack_word(uint32_t w, float (&x)[2]) {  // bf16 -> fp32 is a 16-bit shift
    x[0] = __uint_as_float(w << 16);
    x[1] = __uint_as_float(w & 0xffff0000u);
  }
  static __device__ __forceinline__ uint32_t pack_word(const float (&x)[2]) {
    __nv_bfloat162 h = __floats2bfloat162_rn(x[0], x[1]);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  static __device__ __forceinline__ void unpack(uint4 r, float (&x)[8]) {
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {  // bf16 -> fp32 is a 16-bit shift
      x[2 * i] = __uint_as_float(w[i] << 16);
      x[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
  static __device__ __forceinline__ uint4 pack(const float (&x)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
      __nv_bfloat162 h = __floats2bfloat162_rn(x[2 * i], x[2 * i + 1]);
      w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
  }
  static __device__ __forceinline__ float load1(const __nv_bfloat16* p) { return __bfloat162float(*p); }
  static __device__ __forceinline__ void store1(__nv_bfloat16* p, float x) { *p = __float2bfloat16_rn(x); }
  // The Kahan tail (g <- p ; p <- p + k ; g <- g - p ; k <- k + g) on two packed elements at once.  Each of the
  // three ops takes two values of the storage type and rounds to the storage type; rounding the exact sum
  // directly gives what the fp32 sum rounded again gives (a 24-bit intermediate is more than twice the 8 or
  // 11 bits of the operands plus two, the condition under which double rounding of a sum is harmless), so the
  // native packed instructions reproduce the fp32 sequence bit for bit at a quarter of the instructions.
  static __device__ __forceinline__ void kahan2(uint32_t& p, uint32_t& k) {
    uint32_t np, err;
    asm("add.rn.bf16x2 %0, %1, %2;" : "=r"(np) : "r"(p), "r"(k));
    asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(err) : "r"(p), "r"(np));
    asm("add.rn.bf16x2 %0, %1, %2;" : "=r"(k) : "r"(k), "r"(err));
    p = np;
  }
};
template <> struct Pack<__half> {
  static constexpr int EPW = 2;
  static __device__ __forceinline__ void unpack_word(uint32_t w, float (&x)[2]) {
    float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w));
    x[0] = f.x; x[1] = f.y;
  }
  static __device__ __forceinline__ uint32_t pack_word(const float (&x)[2]) {
    __half2 h = __floats2half2_rn(x[0], x[1]);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  static __device__ __forceinline__ void unpack(uint4 r, float (&x)[8]) {
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
      float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
      x[2 * i] = f.x; x[2 * i + 1] = f.y;
    }
  }
  static __device__ __forceinline__ uint4 pack(const float (&x)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
      __half2 h = __floats2half2_rn(x[2 * i], x[2 * i + 1]);
      w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
  }
  static __device__ __forceinline__ float load1(const __half* p) { return __half2float(*p); }
  static __device__ __forceinline__ void store1(__half* p, float x) { *p = __float2half_rn(x); }
  static __device__ __forceinline__ void kahan2(uint32_t& p, uint32_t& k) {  // see Pack<__nv_bfloat16>::kahan2
    uint32_t np, err;
    asm("add.rn.f16x2 %0, %1, %2;" : "=r"(np) : "r"(p), "r"(k));
    asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(err) : "r"(p), "r"(np));
    asm("add.rn.f16x2 %0, %1, %2;" : "=r"(k) : "r"(k), "r"(err));
    p = np;
  }
};

// streaming 16-byte accesses: every byte is touched once per step
template <typename T> __device__ __forceinline__ uint4 ldv(const T* p) { return __ldcs(reinterpret_cast<const uint4*>(p)); }
template <typename T> __device__ __forceinline__ void stv(T* p, uint4 v) { __stcs(reinterpret_cast<uint4*>(p), v); }

// ---------------------------------------------------------------------------------------------
// scalar-weight lerp, at::native::lerp: |w| < 0.5 ? a + w*(b-a) : b - (b-a)*(1-w), multiply and add
// fused.  Both branches are one fma of d = b-a: fma(d, w, a) or fma(d, -(1-w), b).
// ---------------------------------------------------------------------------------------------
struct Lerp {
  float x;  // w when |w| < 0.5, else -(1-w)
  int low;  // |w| < 0.5
};
__device__ __forceinline__ float lerp_op(float a, float b, const Lerp& l) {
  return __fmaf_rn(__fsub_rn(b, a), l.x, l.low ? a : b);
}

// ---------------------------------------------------------------------------------------------
// tile location
// ---------------------------------------------------------------------------------------------
struct Span {
  int tensor;       // index within the table
  long long begin;  // first element of this block's tile within the tensor
  int len;          // elements in this tile (<= tile size)
};

// `block_elems` = elements one block covers.  s.len is the number of elements of the tensor left
// from s.begin, capped at block_elems.
template <class Table>
__device__ __forceinline__ Span locate(const Table& tab, int block, int block_elems) {
  int t = tab.bucket_tensor[block >> tab.bucket_shift];
  while (tab.tile_start[t + 1] <= block) ++t;  // also skips empty tensors
  Span s;
  s.tensor = t;
  s.begin = (long long)(block - tab.tile_start[t]) * block_elems;
  const long long rem = tab.numel[t] - s.begin;
  s.len = rem < block_elems ? (int)rem : block_elems;
  return s;
}

// Fetches the block's base pointers (advanced to the tile) and reports whether every present list
// is 16-byte aligned there; tile offsets are multiples of 16 bytes, so only the tensors' base
// addresses decide.  The entry of a list that is absent (NULL) is meaningless and never dereferenced:
// an op neither reads nor writes a list the launch did not get.
template <typename T, int NL, class Table>
__device__ __forceinline__ bool tile_pointers(const Table& tab, const Span& s, T* (&p)[NL]) {
  uint32_t bits = 0;
#pragma unroll
  for (int l = 0; l < NL; l++) {
    T* base = reinterpret_cast<T*>(tab.ptr[l][s.tensor]);
    bits |= (uint32_t)reinterpret_cast<uintptr_t>(base);
    p[l] = base + s.begin;
  }
  return (bits & 15) == 0;
}

// ---------------------------------------------------------------------------------------------
// Peer push: the fused form of "step, then all-gather the updated parameters".  Every rank holds
// the parameter buffer at its own virtual address; `delta[j]` is the byte distance from this rank's
// copy to peer j's copy as mapped into this process (symmetric memory over NVLink).  A block that
// has just produced an updated parameter vector stores it locally and, with plain st.global, at the
// same offset in each peer's copy, so the exchange rides along with the step tile by tile.  Plain
// peer stores only, no waits on other ranks inside the kernel (the ranks meet in a
// tiny stream-ordered collective after the launch).
// ---------------------------------------------------------------------------------------------
constexpr int kMaxPeers = 7;
struct PeerPush {
  int n;
  long long delta[kMaxPeers];
};
// Blocks start their round over the peers at different peers (block index modulo the peer count), so
// that the SMs do not all store to the same peer at the same moment.
template <typename T>
__device__ __forceinline__ void push_vec(const PeerPush& push, T* local, uint4 v) {
  const int n = push.n;
  int j = (int)(blockIdx.x % (unsigned)n);
  for (int c = 0; c < n; c++) {
    *reinterpret_cast<uint4*>(reinterpret_cast<char*>(local) + push.delta[j]) = v;
    if (++j == n) j = 0;
  }
}
template <typename T>
__device__ __forceinline__ void push_one(const PeerPush& push, T* local, T v) {
  for (int j = 0; j < push.n; j++) *reinterpret_cast<T*>(reinterpret_cast<char*>(local) + push.delta[j]) = v;
}

// Peer pull: the fused form of "reduce-scatter the gradients, then step".  Every rank keeps its own
// full gradient buffer in memory the others can read; `delta[r]` is the byte distance from this
// rank's buffer to rank r's (0 for this rank itself), for r = 0..n-1 in rank order.  A block loads
// the gradient vector of its tile from all n ranks (all loads issued before the first is used), adds
// them in fp32 in rank order, multiplies by `scale` (1/n for a mean) and rounds once to the storage
// type; the optimizer's arithmetic then sees that value as its gradient.  The reduced gradient
// exists only in registers.  Plain peer loads, no waits on other ranks inside the kernel: the caller
// orders the ranks before the launch (their gradients must be complete) and after it (before the
// buffers are overwritten).
constexpr int kMaxRanks = 8;
struct PeerPull {
  int n;
  float scale;
  long long delta[kMaxRanks];
};
template <typename T> struct Pack;  // defined above
// NR = compile-time bound on the ranks (2, 4 or 8): it sizes the registers that hold the vectors in
// flight, and with them how many blocks fit on an SM — few ranks need many resident threads to keep
// NVLink busy, many ranks need few.
template <typename T, int NR>
__device__ __forceinline__ uint4 pull_vec(const PeerPull& pull, const T* local) {
  constexpr int N = VecN<T>::N;
  uint4 raw[NR];
#pragma unroll
  for (int r = 0; r < NR; r++)
    if (r < pull.n) raw[r] = *reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(local) + pull.delta[r]);
  float acc[N];
  Pack<T>::unpack(raw[0], acc);
#pragma unroll
  for (int r = 1; r < NR; r++) {
    if (r < pull.n) {
      float x[N];
      Pack<T>::unpack(raw[r], x);
#pragma unroll
      for (int j = 0; j < N; j++) acc[j] = __fadd_rn(acc[j], x[j]);
    }
  }
#pragma unroll
  for (int j = 0; j < N; j++) acc[j] = rnd<T>(__fmul_rn(acc[j], pull.scale));
  return Pack<T>::pack(acc);
}
template <typename T>
__device__ __forceinline__ float pull_one(const PeerPull& pull, const T* local) {
  float acc = 0.f;
  for (int r = 0; r < pull.n; r++) {
    const float x = Pack<T>::load1(reinterpret_cast<const T*>(reinterpret_cast<const char*>(local) + pull.delta[r]));
    acc = r == 0 ? x : __fadd_rn(acc, x);
  }
  return rnd<T>(__fmul_rn(acc, pull.scale));
}

// ---------------------------------------------------------------------------------------------
// Generic element-wise machinery.  An Op describes one optimizer variant:
//   NL, U                     number of tensor lists, vectors per thread per list in a full tile
//   Args                      uniform scalars of the launch
//   Ctx / context(...)        per-tile values (per-tensor scalars for StableAdamW, empty otherwise)
//   reads(l, args)            list l is loaded        (uniform across the launch)
//   writes(l, args)           list l is stored back   (uniform across the launch)
//   elem<T, TAIL, L2>(e, args, ctx)   the arithmetic for ONE element; e[l] is the element of list l as fp32
//   kHasL2 / l2(args)         the op has an L2 weight-decay form, and whether this launch is one
//   kPackedTail, kSlotP/K     16-bit storage: whole vectors call elem with TAIL = false and finish with the Kahan tail
//                             on packed pairs of lists kSlotP (parameter) and kSlotK (compensation)
//   kPostTail / post_tail     what remains to be done to the parameter after that tail
//   kSumSlot                  index of an e[] slot whose values compute_vec sums up (-1: none)
//   kMinBlocks                blocks that must fit on one SM (register cap for the compiler)
//   kWholeTileBranch          give whole tiles their own straight-line branch (a code-generation choice
//                             made per op by measurement: +8 % for Lion and StableAdamW, -7 % for Adam)
//   kPush                     also store updated parameters into the peers' copies (Args has .push)
//   kPull                     0, or the rank bound (2/4/8) of a launch whose gradients are the scaled sum of all
//                             ranks' gradient buffers (Args has .pull)
// ---------------------------------------------------------------------------------------------
struct NoCtx {};

template <int NL> struct Vecs { uint4 r[NL]; };

template <typename T, class Op>
__device__ __forceinline__ void load_vec(Vecs<Op::NL>& v, T* const (&p)[Op::NL], int i, const typename Op::Args& a) {
#pragma unroll
  for (int l = 0; l < Op::NL; l++) {
    if constexpr (Op::kPull) {  // list 1 is the gradient list in every op that can pull
      if (l == 1) {
        v.r[1] = pull_vec<T, Op::kPull>(a.pull, p[1] + i);
        continue;
      }
    }
    if (Op::reads(l, a)) v.r[l] = ldv(p[l] + i);
  }
}

template <typename T, class Op>
__device__ __forceinline__ void store_vec(const Vecs<Op::NL>& v, T* const (&p)[Op::NL], int i, const typename Op::Args& a) {
#pragma unroll
  for (int l = 0; l < Op::NL; l++)
    if (Op::writes(l, a)) stv(p[l] + i, v.r[l]);
  if constexpr (Op::kPush) {  // list 0 is the parameter list in every op that can push
    if (Op::writes(0, a)) push_vec(a.push, p[0] + i, v.r[0]);
  }
}

__device__ __forceinline__ uint32_t& word_of(uint4& v, int i) { return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w; }

// One 16-byte vector per list, 32-bit word by word: the one (fp32) or two (16-bit types) elements of a
// word are unpacked, run through the op and packed back before the next word is touched, so that few
// values are live at a time; the packed Kahan tail then works on the word in place.
template <typename T, class Op, bool L2>
__device__ __forceinline__ float compute_vec_as(Vecs<Op::NL>& v, const typename Op::Args& a, const typename Op::Ctx& ctx) {
  constexpr int EPW = Pack<T>::EPW;  // elements per word
  constexpr bool PACKED_TAIL = Op::kPackedTail && sizeof(T) == 2;
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < 4; i++) {
    float e[EPW][Op::NL];
#pragma unroll
    for (int l = 0; l < Op::NL; l++) {
      if (Op::reads(l, a)) {
        float x[EPW];
        Pack<T>::unpack_word(word_of(v.r[l], i), x);
#pragma unroll
        for (int j = 0; j < EPW; j++) e[j][l] = x[j];
      } else {
#pragma unroll
        for (int j = 0; j < EPW; j++) e[j][l] = 0.f;
      }
    }
#pragma unroll
    for (int j = 0; j < EPW; j++) {
      Op::template elem<T, !PACKED_TAIL, L2>(e[j], a, ctx);
      if (Op::kSumSlot >= 0) sum += e[j][Op::kSumSlot < 0 ? 0 : Op::kSumSlot];
    }
#pragma unroll
    for (int l = 0; l < Op::NL; l++) {
      if (Op::writes(l, a)) {
        float x[EPW];
#pragma unroll
        for (int j = 0; j < EPW; j++) x[j] = e[j][l];
        word_of(v.r[l], i) = Pack<T>::pack_word(x);
      }
    }
    if constexpr (PACKED_TAIL) {
      uint32_t &pw = word_of(v.r[Op::kSlotP], i), &kw = word_of(v.r[Op::kSlotK], i);
      Pack<T>::kahan2(pw, kw);
      if constexpr (Op::kPostTail) {
        float x[EPW];
        Pack<T>::unpack_word(pw, x);
#pragma unroll
        for (int j = 0; j < EPW; j++) x[j] = Op::template post_tail<T>(x[j], a);
        pw = Pack<T>::pack_word(x);
      }
    }
  }
  return sum;
}

template <typename T, class Op>
__device__ __forceinline__ float compute_vec(Vecs<Op::NL>& v, const typename Op::Args& a, const typename Op::Ctx& ctx) {
  if constexpr (Op::kHasL2) {
    if (Op::l2(a)) return compute_vec_as<T, Op, true>(v, a, ctx);
  }
  return compute_vec_as<T, Op, false>(v, a, ctx);
}

template <typename T, class Op>
__device__ __forceinline__ float scalar_elem(T* const (&p)[Op::NL], int i, const typename Op::Args& a,
                                             const typename Op::Ctx& ctx) {
  float e[Op::NL];
#pragma unroll
  for (int l = 0; l < Op::NL; l++) e[l] = Op::reads(l, a) ? Pack<T>::load1(p[l] + i) : 0.f;
  if constexpr (Op::kPull) e[1] = pull_one<T>(a.pull, p[1] + i);
  if (Op::kHasL2 && Op::l2(a)) Op::template elem<T, true, true>(e, a, ctx);
  else Op::template elem<T, true, false>(e, a, ctx);
#pragma unroll
  for (int l = 0; l < Op::NL; l++)
    if (Op::writes(l, a)) Pack<T>::store1(p[l] + i, e[l]);
  if constexpr (Op::kPush) {
    if (Op::writes(0, a)) push_one(a.push, p[0] + i, p[0][i]);
  }
  return Op::kSumSlot >= 0 ? e[Op::kSumSlot < 0 ? 0 : Op::kSumSlot] : 0.f;
}

// Processes the block's tile; returns this thread's share of the kSumSlot sum (0 without one).
template <typename T, class Op, class Table>
__device__ __forceinline__ double process_tile(const Table& tab, const typename Op::Args& args, Span& s) {
  constexpr int V = VecN<T>::N;
  constexpr int U = Op::U;
  constexpr int TILE = kThreads * U * V;
  s = locate(tab, blockIdx.x, TILE);
  T* p[Op::NL];
  const bool aligned = tile_pointers<T, Op::NL, Table>(tab, s, p);
  const typename Op::Ctx ctx = Op::context(tab, s, args);
  double acc = 0.0;
  int done = 0;
  if (Op::kWholeTileBranch && aligned && s.len == TILE) {
    // a whole tile, as straight-line code ahead of the general loops below (same work; for some ops
    // the compiler's schedule of this form runs measurably faster, for others slower: see kWholeTileBranch)
    Vecs<Op::NL> v[U];
#pragma unroll
    for (int u = 0; u < U; u++) load_vec<T, Op>(v[u], p, (u * kThreads + threadIdx.x) * V, args);
#pragma unroll
    for (int u = 0; u < U; u++) {
      const float part = compute_vec<T, Op>(v[u], args, ctx);
      store_vec<T, Op>(v[u], p, (u * kThreads + threadIdx.x) * V, args);
      if (Op::kSumSlot >= 0) acc += (double)part;
    }
    return acc;
  }
  if (aligned) {
    for (; done + TILE <= s.len; done += TILE) {
      Vecs<Op::NL> v[U];
#pragma unroll
      for (int u = 0; u < U; u++) load_vec<T, Op>(v[u], p, done + (u * kThreads + threadIdx.x) * V, args);
#pragma unroll
      for (int u = 0; u < U; u++) {
        const float part = compute_vec<T, Op>(v[u], args, ctx);
        store_vec<T, Op>(v[u], p, done + (u * kThreads + threadIdx.x) * V, args);
        if (Op::kSumSlot >= 0) acc += (double)part;
      }
    }
    // ragged end of the tensor: whole vectors, then single elements
    const int nvec = (s.len - done) / V;
    for (int i = threadIdx.x; i < nvec; i += kThreads) {
      Vecs<Op::NL> v;
      load_vec<T, Op>(v, p, done + i * V, args);
      const float part = compute_vec<T, Op>(v, args, ctx);
      store_vec<T, Op>(v, p, done + i * V, args);
      if (Op::kSumSlot >= 0) acc += (double)part;
    }
    done += nvec * V;
  }
  for (int i = done + threadIdx.x; i < s.len; i += kThreads) acc += (double)scalar_elem<T, Op>(p, i, args, ctx);
  return acc;
}

// Op::kMinBlocks caps the registers per thread (65536 / (kThreads * kMinBlocks)): residency, not
// per-thread instruction-level parallelism, is what keeps the memory pipeline full here.
template <typename T, class Op, bool SMALL>
__global__ void __launch_bounds__(kThreads, Op::kMinBlocks) mta_kernel(const __grid_constant__ MtaTable<Op::NL, SMALL> tab,
                                                       const __grid_constant__ typename Op::Args args) {
  Span s;
  process_tile<T, Op>(tab, args, s);
}

}  // namespace optimi
