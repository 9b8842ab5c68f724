// Per-element arithmetic of the eight optimizers, as "ops" for the generic multi-tensor kernel.
//
// Every op replays the reference's foreach sequence for its optimizer in registers: each statement
// that ends in rnd<T>(...) is ONE ATen op of that sequence — an fp32 computation followed by a
// rounding to the storage type — in the reference's order, with the fp32 formula the CUDA build of
// that ATen op uses (fused multiply-add for `x + s*y`, correctly rounded sqrt and divide, division
// by a scalar as multiplication by its reciprocal).  Intermediates that the reference keeps in the
// gradient buffer live in registers here, so gradients are never written.
//
// Template flags: KAHAN = Kahan-compensated update (16-bit storage only), UPDATE = false is the
// optimizer-accumulation micro-step (state averages only).
//
// Flags of elem<T, TAIL, L2>: TAIL = false leaves the closing Kahan tail (p += k with the error fed back
// into k) to the caller, who does it on packed pairs (Pack<T>::kahan2) — an op offers this with
// kPackedTail and names the slots with kSlotP / kSlotK; what must still happen to the parameter after
// the tail goes into post_tail (kPostTail).  L2 = true is the launch with L2 weight decay (the gradient
// gains wd*p); otherwise the parameter is multiplied by the launch's decay factor, which is 1 when
// there is no decay (a product with 1 is exact).  Which of the two a launch is, is uniform, so the
// caller branches once per vector (l2(args)) instead of the op testing a mode per element.
#pragma once

#include "mta_common.cuh"

namespace optimi {

enum WdMode : int { kWdNone = 0, kWdDecoupled = 1, kWdL2 = 2 };

// g <- p ; p <- p + k ; g <- g - p ; k <- k + g        (e.g. optimi/adam.py:445-450)
template <typename T>
__device__ __forceinline__ void kahan_tail(float& p, float& k) {
  const float old = p;
  p = rnd<T>(__fadd_rn(p, k));
  const float err = rnd<T>(__fsub_rn(old, p));
  k = rnd<T>(__fadd_rn(k, err));
}

// copy ; sqrt ; add eps                                  (e.g. optimi/adam.py:437-439)
template <typename T>
__device__ __forceinline__ float denominator(float v, float eps) {
  return rnd<T>(__fadd_rn(sqrt_rnd<T>(v), eps));
}

// correctly rounded a / b; for the 16-bit storage types through the one-correction shortcut
template <typename T>
__device__ __forceinline__ float quotient(float a, float b) {
  if constexpr (sizeof(T) == 2) return div16(a, b, rcp_fast(b));
  else return __fdiv_rn(a, b);
}

// addcdiv: x + value * (a / b)
template <typename T>
__device__ __forceinline__ float addcdiv_op(float x, float a, float b, float value) {
  return __fmaf_rn(value, quotient<T>(a, b), x);
}

// lerp ; mul ; addcmul                                    (e.g. optimi/adam.py:431-434)
template <typename T>
__device__ __forceinline__ void adam_moments(float& m, float& v, float g, const Lerp& l1, float beta2_hat, float beta2_comp) {
  m = rnd<T>(lerp_op(m, g, l1));
  v = rnd<T>(__fmul_rn(v, beta2_hat));
  v = rnd<T>(__fmaf_rn(beta2_comp, __fmul_rn(g, g), v));
}

// A value that goes nowhere but into its list's store needs no rounding of its own: packing it for the store
// (Pack<T>::pack_word, store1) IS that rounding.  ROUND = false marks such a last op; the packed Kahan tail
// counts as a store here, because it starts from the packed words.
template <typename T, bool ROUND>
__device__ __forceinline__ float rnd_if(float x) { return ROUND ? rnd<T>(x) : x; }

// ROUND_P: the decayed parameter is used again by this element's arithmetic (false: it only goes to the tail / store)
template <typename T, bool L2, bool ROUND_P>
__device__ __forceinline__ void weight_decay(float& p, float& g, float wd) {
  if (L2) g = rnd<T>(__fmaf_rn(wd, p, g));
  else p = rnd_if<T, ROUND_P>(__fmul_rn(p, wd));
}

struct OpBase {
  using Ctx = NoCtx;
  static constexpr int kSumSlot = -1;
  static constexpr int kMinBlocks = 12;  // <= 40 registers per thread at 128 threads
  static constexpr bool kPush = false;
  static constexpr int kPull = 0;
  static constexpr bool kWholeTileBranch = false;
  static constexpr int kGradSlot = 1;  // the list that holds the gradients
  static constexpr bool kPackedTail = false, kPostTail = false, kHasL2 = false;
  static constexpr int kSlotP = 0, kSlotK = 0;
  template <class Args>
  static __device__ __forceinline__ bool l2(const Args&) { return false; }
  template <class Table, class Args>
  static __device__ __forceinline__ NoCtx context(const Table&, const Span&, const Args&) { return NoCtx{}; }
  template <typename T, class Args>
  static __device__ __forceinline__ float post_tail(float p, const Args&) { return p; }
};

// ---------------------------------------------------------------------------------------------
// Adam / AdamW                                       lists: 0 p, 1 g, 2 m, 3 v, 4 k (kahan)
// optimi/adam.py:424-453
// ---------------------------------------------------------------------------------------------
struct AdamArgs {
  Lerp l1;
  float beta2_hat, beta2_comp, wd, eps, neg_lr;
  int wd_mode;
};

template <bool KAHAN, bool UPDATE>
struct AdamOp : OpBase {
  static constexpr int NL = 5, U = 1;
  static constexpr bool kPackedTail = KAHAN && UPDATE, kHasL2 = UPDATE;
  static constexpr int kSlotP = 0, kSlotK = 4;
  using Args = AdamArgs;
  static __device__ __forceinline__ bool l2(const Args& a) { return a.wd_mode == kWdL2; }
  static __device__ __forceinline__ bool reads(int l, const Args&) { return l == 0 ? UPDATE : l == 4 ? KAHAN : true; }
  static __device__ __forceinline__ bool writes(int l, const Args&) { return l == 0 ? UPDATE : l == 4 ? KAHAN : l != 1; }
  template <typename T, bool TAIL, bool L2>
  static __device__ __forceinline__ void elem(float (&e)[NL], const Args& a, const NoCtx&) {
    float &p = e[0], &g = e[1], &m = e[2], &v = e[3], &k = e[4];
    if (UPDATE) weight_decay<T, L2, !KAHAN || TAIL>(p, g, a.wd);
    adam_moments<T>(m, v, g, a.l1, a.beta2_hat, a.beta2_comp);
    if (UPDATE) {
      const float den = denominator<T>(v, a.eps);
      if (KAHAN) {
        k = rnd_if<T, TAIL>(addcdiv_op<T>(k, m, den, a.neg_lr));
        if (TAIL) kahan_tail<T>(p, k);
      } else {
        p = addcdiv_op<T>(p, m, den, a.neg_lr);  // rounded by the store
      }
    }
  }
};

// Any op whose list 0 is the parameter list and list 1 the gradient list, with the peer push added
// to its stores and, when PULL, the gradient replaced by the scaled sum over all ranks' gradients.
template <class BaseArgs>
struct PeerArgs {
  BaseArgs base;
  PeerPush push;
  PeerPull pull;
};

template <class Base, int PULL>  // PULL: 0 = push only, else the rank bound 2, 4 or 8
struct PeerOp {
  static constexpr int NL = Base::NL, U = Base::U, kSumSlot = Base::kSumSlot;
  // Remote loads take microseconds: what keeps NVLink busy is many resident threads, each with its
  // gradient vectors in flight (two vectors per thread at half the residency was measured slower;
  // beyond ~900 resident threads per SM nothing is gained: the link direction that carries both the
  // peers' pushes and this rank's read responses is then the limit).  The register cap loosens as
  // the rank bound, and with it the vectors held, grows.
  static constexpr int kMinBlocks = PULL == 0 ? (Base::kMinBlocks > 2 ? Base::kMinBlocks - 2 : 1)
                                    : PULL == 2 ? (Base::kMinBlocks > 3 ? Base::kMinBlocks - 3 : 1)
                                    : PULL == 4 ? (Base::kMinBlocks > 4 ? Base::kMinBlocks - 4 : 1)
                                                : (Base::kMinBlocks > 6 ? Base::kMinBlocks - 6 : 1);
  static constexpr bool kPush = true;
  static constexpr int kPull = PULL;
  static constexpr bool kWholeTileBranch = false;
  static constexpr bool kPackedTail = Base::kPackedTail, kPostTail = Base::kPostTail, kHasL2 = Base::kHasL2;
  static constexpr int kSlotP = Base::kSlotP, kSlotK = Base::kSlotK;
  using Args = PeerArgs<typename Base::Args>;
  static __device__ __forceinline__ bool l2(const Args& a) { return Base::l2(a.base); }
  using Ctx = typename Base::Ctx;
  template <class Table>
  static __device__ __forceinline__ Ctx context(const Table& tab, const Span& s, const Args& a) { return Base::context(tab, s, a.base); }
  static __device__ __forceinline__ bool reads(int l, const Args& a) { return Base::reads(l, a.base); }
  static __device__ __forceinline__ bool writes(int l, const Args& a) { return Base::writes(l, a.base); }
  template <typename T, bool TAIL, bool L2>
  static __device__ __forceinline__ void elem(float (&e)[NL], const Args& a, const Ctx& ctx) {
    Base::template elem<T, TAIL, L2>(e, a.base, ctx);
  }
  template <typename T>
  static __device__ __forceinline__ float post_tail(float p, const Args& a) { return Base::template post_tail<T>(p, a.base); }
};

// Any op with its gradients multiplied, as they are loaded, by one fp32 factor read from device
// memory: g <- round(g * factor), the arithmetic of `torch._foreach_mul_(grads, factor_tensor)`
// (what clip_grad_norm_ and GradScaler.unscale_ do to the gradients in a pass of their own).  The
// scaled gradient exists only in registers; the gradient buffer is not written.
template <class BaseArgs>
struct ScaledArgs {
  BaseArgs base;
  const float* factor;  // device
};

template <class Base>
struct ScaledOp {
  static constexpr int NL = Base::NL, U = Base::U, kSumSlot = Base::kSumSlot, kMinBlocks = Base::kMinBlocks;
  static constexpr bool kPush = false;
  static constexpr int kPull = 0;
  static constexpr bool kWholeTileBranch = Base::kWholeTileBranch;
  static constexpr int kGradSlot = Base::kGradSlot;
  static constexpr bool kPackedTail = Base::kPackedTail, kPostTail = Base::kPostTail, kHasL2 = Base::kHasL2;
  static constexpr int kSlotP = Base::kSlotP, kSlotK = Base::kSlotK;
  using Args = ScaledArgs<typename Base::Args>;
  static __device__ __forceinline__ bool l2(const Args& a) { return Base::l2(a.base); }
  struct Ctx {
    typename Base::Ctx base;
    float factor;
  };
  template <class Table>
  static __device__ __forceinline__ Ctx context(const Table& tab, const Span& s, const Args& a) {
    return Ctx{Base::context(tab, s, a.base), __ldg(a.factor)};
  }
  static __device__ __forceinline__ bool reads(int l, const Args& a) { return Base::reads(l, a.base); }
  static __device__ __forceinline__ bool writes(int l, const Args& a) { return Base::writes(l, a.base); }
  template <typename T, bool TAIL, bool L2>
  static __device__ __forceinline__ void elem(float (&e)[NL], const Args& a, const Ctx& ctx) {
    e[kGradSlot] = rnd<T>(__fmul_rn(e[kGradSlot], ctx.factor));
    Base::template elem<T, TAIL, L2>(e, a.base, ctx.base);
  }
  template <typename T>
  static __device__ __forceinline__ float post_tail(float p, const Args& a) { return Base::template post_tail<T>(p, a.base); }
};

// ---------------------------------------------------------------------------------------------
// Sum of squares of a gradient list (the first pass of a gradient-norm clip)
// lists: 0 g, 1 (pseudo, no memory) carries g^2 out for the tile sum
// ---------------------------------------------------------------------------------------------
struct SumSqArgs {};
struct SumSqOp : OpBase {
  // one stream, read only: four vectors per thread in flight (8 KB per block), or the per-block cost
  // of the reduction dominates (one vector per thread measured 2.9 TB/s)
  static constexpr int NL = 2, U = 4;
  static constexpr int kSumSlot = 1;
  static constexpr int kMinBlocks = 12;
  static constexpr bool kWholeTileBranch = true;
  static constexpr int kGradSlot = 0;
  using Args = SumSqArgs;
  static __device__ __forceinline__ bool reads(int l, const Args&) { return l == 0; }
  static __device__ __forceinline__ bool writes(int, const Args&) { return false; }
  template <typename T, bool TAIL, bool L2>
  static __device__ __forceinline__ void elem(float (&e)[NL], const Args&, const NoCtx&) {
    e[1] = __fmul_rn(e[0], e[0]);
  }
};

// ---------------------------------------------------------------------------------------------
// RAdam and Ranger              lists: 0 p, 1 g, 2 m, 3 v, 4 k, 5 la (slow weights, Ranger only)
// optimi/radam.py:438-479, optimi/ranger.py:498-561
// ---------------------------------------------------------------------------------------------
struct RangerArgs {
  Lerp l1;
  float beta2_hat, beta2_comp, wd, eps, neg_lr;  // neg_lr = -lr*rect when use_rect
  float alpha;
  int wd_mode, use_rect, lookahead;
};

// LOOK = true only for the launches of a Ranger step that falls on a lookahead step; RAdam and the
// other Ranger steps never touch the slow weights and keep Adam's register budget.
template <bool KAHAN, bool UPDATE, bool LOOK>
struct RangerOp : OpBase {
  static constexpr int NL = 6, U = 1;
  // six streams: <= 64 registers; five: as Adam (without the packed Kahan tail a little more is live)
  static constexpr int kMinBlocks = LOOK ? 8 : KAHAN ? OpBase::kMinBlocks : 10;
  // a lookahead step goes on after the tail (a second compensated sum into the slow weights): it keeps the fp32 form
  static constexpr bool kPackedTail = KAHAN && UPDATE && !LOOK, kHasL2 = UPDATE;
  static constexpr int kSlotP = 0, kSlotK = 4;
  using Args = RangerArgs;
  static __device__ __forceinline__ bool l2(const Args& a) { return a.wd_mode == kWdL2; }
  static __device__ __forceinline__ bool reads(int l, const Args&) {
    return l == 0 ? UPDATE : l == 4 ? KAHAN : l == 5 ? (UPDATE && LOOK) : true;
  }
  static __device__ __forceinline__ bool writes(int l, const Args& a) { return l != 1 && reads(l, a); }
  template <typename T, bool TAIL, bool L2>
  static __device__ __forceinline__ void elem(float (&e)[NL], const Args& a, const NoCtx&) {
    float &p = e[0], &g = e[1], &m = e[2], &v = e[3], &k = e[4], &la = e[5];
    constexpr bool kMore = LOOK || (KAHAN && TAIL);  // the step's result is used again before it is stored
    if (UPDATE) weight_decay<T, L2, !KAHAN || kMore>(p, g, a.wd);
    adam_moments<T>(m, v, g, a.l1, a.beta2_hat, a.beta2_comp);
    if (UPDATE) {
      float x = KAHAN ? k : p;
      if (a.use_rect) x = rnd_if<T, kMore>(addcdiv_op<T>(x, m, denominator<T>(v, a.eps), a.neg_lr));
      else x = rnd_if<T, kMore>(__fmaf_rn(a.neg_lr, m, x));
      if (KAHAN) {
        k = x;
        if (TAIL || LOOK) kahan_tail<T>(p, k);
        if (LOOK) {  // optimi/ranger.py:537-549
          const float diff = rnd<T>(__fsub_rn(p, la));
          k = rnd<T>(__fmaf_rn(a.alpha, diff, k));
          kahan_tail<T>(la, k);
          p = la;
        }
      } else {
        p = x;
        if (LOOK) {  // optimi/ranger.py:559-561
          p = rnd<T>(__fsub_rn(p, la));
          la = rnd<T>(__fmaf_rn(a.alpha, p, la));
          p = la;
        }
      }
    }
  }
};

template <bool KAHAN, bool UPDATE> using RadamOp = RangerOp<KAHAN, UPDATE, false>;
template <bool KAHAN, bool UPDATE> using RangerLookOp = RangerOp<KAHAN, UPDATE, true>;

// ---------------------------------------------------------------------------------------------
// Lion                                                        lists: 0 p, 1 g, 2 m, 3 k
// optimi/lion.py:354-380
// ---------------------------------------------------------------------------------------------
struct LionArgs {
  Lerp l1, l2;
  float wd, neg_lr;
  int wd_mode;
};

template <bool KAHAN, bool UPDATE>
struct LionOp : OpBase {
  static constexpr int NL = 4, U = 1;
  static constexpr bool kWholeTileBranch = true;
  static constexpr bool kPackedTail = KAHAN && UPDATE;
  static constexpr int kSlotP = 0, kSlotK = 3;
  using Args = LionArgs;
  static __device__ __forceinline__ bool reads(int l, const Args&) { return l == 0 ? UPDATE : l == 3 ? KAHAN : true; }
  static __device__ __forceinline__ bool writes(int l, const Args& a) { return l != 1 && reads(l, a); }
  template <typename T, bool TAIL, bool L2>
  static __device__ __forceinline__ void elem(float (&e)[NL], const Args& a, const NoCtx&) {
    float &p = e[0], &g = e[1], &m = e[2], &k = e[3];
    float u = 0.f;
    if (UPDATE) {
      p = rnd_if<T, !KAHAN || TAIL>(__fmul_rn(p, a.wd));  // the decay factor, 1 without decay
      u = rnd<T>(lerp_op(m, g, a.l1));
      u = u > 0.f ? 1.f : (u < 0.f ? -1.f : 0.f);  // sign; NaN -> 0 like (0 < u) - (u < 0)
    }
    m = lerp_op(m, g, a.l2);  // rounded by the store
    if (UPDATE) {
      if (KAHAN) {
        k = rnd_if<T, TAIL>(__fmaf_rn(a.neg_lr, u, k));
        if (TAIL) kahan_tail<T>(p, k);
      } else {
        p = __fmaf_rn(a.neg_lr, u, p);  // rounded by the store
      }
    }
  }
};

// ---------------------------------------------------------------------------------------------
// SGD                                     lists: 0 p, 1 g, 2 m (absent when momentum == 0), 3 k
// optimi/sgd.py:389-421
// ---------------------------------------------------------------------------------------------
struct SgdArgs {
  Lerp damp;  // weight 1 - momentum
  float momentum, wd, neg_lr;
  int wd_mode, has_momentum, dampening;
};

template <bool KAHAN, bool UPDATE>
struct SgdOp : OpBase {
  static constexpr int NL = 4, U = 1;
  // no L2 variant here: with only four streams the kernel sits at the DRAM ceiling, and the leaner variant form,
  // which fits 32 registers and so sixteen resident blocks, measured 1 % slower than testing the mode per element
  static constexpr bool kPackedTail = KAHAN && UPDATE;
  static constexpr int kSlotP = 0, kSlotK = 3;
  using Args = SgdArgs;
  static __device__ __forceinline__ bool reads(int l, const Args& a) {
    return l == 0 ? UPDATE : l == 2 ? a.has_momentum != 0 : l == 3 ? KAHAN : true;
  }
  static __device__ __forceinline__ bool writes(int l, const Args& a) { return l != 1 && reads(l, a); }
  template <typename T, bool TAIL, bool L2>
  static __device__ __forceinline__ void elem(float (&e)[NL], const Args& a, const NoCtx&) {
    float &p = e[0], &g = e[1], &m = e[2], &k = e[3];
    if (UPDATE) {
      if (a.wd_mode == kWdDecoupled) p = rnd<T>(__fmul_rn(p, a.wd));
      else if (a.wd_mode == kWdL2) g = rnd<T>(__fmaf_rn(a.wd, p, g));
    }
    float upd = g;
    if (a.has_momentum) {
      if (a.dampening) {
        m = rnd<T>(lerp_op(m, g, a.damp));
      } else {
        m = rnd<T>(__fmul_rn(m, a.momentum));
        m = rnd<T>(__fadd_rn(m, g));
      }
      upd = m;
    }
    if (UPDATE) {
      if (KAHAN) {
        k = rnd<T>(__fmaf_rn(a.neg_lr, upd, k));
        if (TAIL) kahan_tail<T>(p, k);
      } else {
        p = rnd<T>(__fmaf_rn(a.neg_lr, upd, p));
      }
    }
  }
};

// ---------------------------------------------------------------------------------------------
// Adan     lists: 0 p, 1 g, 2 m (exp_avg), 3 d (exp_avg_diff), 4 q (exp_avg_sq), 5 pg (-g_prev), 6 k
// optimi/adan.py:500-546
// ---------------------------------------------------------------------------------------------
struct AdanArgs {
  Lerp l1, l2;
  float beta2, beta3_hat, beta3_comp, eps, neg_lr, neg_lr_beta2;
  float wd_mul;  // adam_wd: factor 1 - lr*wd ; Adan style: fp32 reciprocal of 1 + lr*wd
  int wd_mode;   // 0 none, 1 adam_wd (multiply before the step), 2 Adan style (divide after the step)
};

template <bool KAHAN, bool UPDATE>
struct AdanOp : OpBase {
  static constexpr int NL = 7, U = 1;
  static constexpr int kMinBlocks = 8;  // seven streams: 64 registers, the most that still compiles without spills
  static constexpr bool kPackedTail = KAHAN && UPDATE, kPostTail = KAHAN && UPDATE;
  static constexpr int kSlotP = 0, kSlotK = 6;
  using Args = AdanArgs;
  // Adan-style weight decay divides the parameter after the step (optimi/adan.py:546)
  template <typename T>
  static __device__ __forceinline__ float post_tail(float p, const Args& a) {
    return a.wd_mode == 2 ? __fmul_rn(p, a.wd_mul) : p;  // rounded when it is packed for the store
  }
  static __device__ __forceinline__ bool reads(int l, const Args&) { return l == 0 ? UPDATE : l == 6 ? KAHAN : true; }
  static __device__ __forceinline__ bool writes(int l, const Args& a) { return l != 1 && reads(l, a); }
  template <typename T, bool TAIL, bool L2>
  static __device__ __forceinline__ void elem(float (&e)[NL], const Args& a, const NoCtx&) {
    float &p = e[0], &g = e[1], &m = e[2], &d = e[3], &q = e[4], &pg = e[5], &k = e[6];
    float diff = rnd<T>(__fadd_rn(pg, g));
    m = rnd<T>(lerp_op(m, g, a.l1));
    d = rnd<T>(lerp_op(d, diff, a.l2));
    diff = rnd<T>(__fmul_rn(diff, a.beta2));
    diff = rnd<T>(__fadd_rn(diff, g));
    q = rnd<T>(__fmul_rn(q, a.beta3_hat));
    q = rnd<T>(__fmaf_rn(a.beta3_comp, __fmul_rn(diff, diff), q));
    pg = -g;
    if (UPDATE) {
      const float den = denominator<T>(q, a.eps);
      if (a.wd_mode == 1) p = rnd_if<T, !KAHAN || TAIL>(__fmul_rn(p, a.wd_mul));
      // both quotients share the denominator, and with it the reciprocal of the shortcut
      float qm, qd;
      if constexpr (sizeof(T) == 2) {
        const float y = rcp_fast(den);
        qm = div16(m, den, y);
        qd = div16(d, den, y);
      } else {
        qm = __fdiv_rn(m, den);
        qd = __fdiv_rn(d, den);
      }
      if (KAHAN) {
        k = rnd<T>(__fmaf_rn(a.neg_lr, qm, k));
        k = rnd_if<T, TAIL>(__fmaf_rn(a.neg_lr_beta2, qd, k));
        if (TAIL) {
          kahan_tail<T>(p, k);
          p = post_tail<T>(p, a);
        }
      } else {
        p = rnd<T>(__fmaf_rn(a.neg_lr, qm, p));
        p = rnd<T>(__fmaf_rn(a.neg_lr_beta2, qd, p));
        if (a.wd_mode == 2) p = __fmul_rn(p, a.wd_mul);  // rounded by the store
      }
    }
  }
};

// ---------------------------------------------------------------------------------------------
// StableAdamW, pass A (moments + per-tile sum)       lists: 0 g, 1 m, 2 v, 3 r (pseudo, no memory)
// optimi/stableadamw.py:499-506.  e[3] carries g^2 / max(v, eps^2) out for the tile sum.
// ---------------------------------------------------------------------------------------------
struct StableMomentsArgs {
  Lerp l1;
  float beta2_hat, beta2_comp, eps_sq;  // eps_sq: eps^2 rounded to the storage type
};

constexpr int kStableMinBlocks = 12;  // both StableAdamW passes fit 40 registers: twelve blocks per SM

template <bool REDUCE>
struct StableMomentsOp : OpBase {
  static constexpr int NL = 4, U = 1;
  static constexpr int kMinBlocks = kStableMinBlocks;
  static constexpr bool kWholeTileBranch = true;
  static constexpr int kGradSlot = 0;
  static constexpr int kSumSlot = REDUCE ? 3 : -1;
  using Args = StableMomentsArgs;
  static __device__ __forceinline__ bool reads(int l, const Args&) { return l != 3; }
  static __device__ __forceinline__ bool writes(int l, const Args&) { return l == 1 || l == 2; }
  template <typename T, bool TAIL, bool L2>
  static __device__ __forceinline__ void elem(float (&e)[NL], const Args& a, const NoCtx&) {
    float &g = e[0], &m = e[1], &v = e[2];
    adam_moments<T>(m, v, g, a.l1, a.beta2_hat, a.beta2_comp);
    if (REDUCE) {
      const float x = fmaxf(v, a.eps_sq);  // the larger of two values of the storage type: no rounding needed
      const float gg = rnd<T>(__fmul_rn(g, g));
      e[3] = rnd<T>(quotient<T>(gg, x));  // div (optimi/stableadamw.py:506), correctly rounded like ATen's
    }
  }
};

// ---------------------------------------------------------------------------------------------
// StableAdamW, pass B (parameter update)                    lists: 0 p, 1 m, 2 v, 3 k
// optimi/stableadamw.py:522-544.  The clipped -lr and the weight-decay factor are per tensor.
// ---------------------------------------------------------------------------------------------
struct StableUpdateArgs {
  const float2* tensor_scalars;  // per tensor: x = -lr / max(1, rms), y = weight-decay factor
  float eps;
  int has_wd;
};

template <bool KAHAN>
struct StableUpdateOp {
  static constexpr int NL = 4, U = 1;
  static constexpr int kSumSlot = -1;
  static constexpr int kMinBlocks = kStableMinBlocks;
  static constexpr bool kPush = false;
  static constexpr int kPull = 0;
  static constexpr bool kWholeTileBranch = true;
  static constexpr bool kPackedTail = KAHAN, kPostTail = false, kHasL2 = false;
  static constexpr int kSlotP = 0, kSlotK = 3;
  using Args = StableUpdateArgs;
  static __device__ __forceinline__ bool l2(const Args&) { return false; }
  using Ctx = float2;
  template <typename T>
  static __device__ __forceinline__ float post_tail(float p, const Args&) { return p; }
  template <class Table>
  static __device__ __forceinline__ float2 context(const Table& tab, const Span& s, const Args& a) {
    return a.tensor_scalars[tab.tensor_base + s.tensor];
  }
  static __device__ __forceinline__ bool reads(int l, const Args&) { return l == 3 ? KAHAN : true; }
  static __device__ __forceinline__ bool writes(int l, const Args&) { return l == 0 || (l == 3 && KAHAN); }
  template <typename T, bool TAIL, bool L2>
  static __device__ __forceinline__ void elem(float (&e)[NL], const Args& a, const float2& sc) {
    float &p = e[0], &m = e[1], &v = e[2], &k = e[3];
    if (a.has_wd) p = rnd_if<T, !KAHAN || TAIL>(__fmul_rn(p, sc.y));
    const float den = denominator<T>(v, a.eps);
    if (KAHAN) {
      k = rnd_if<T, TAIL>(addcdiv_op<T>(k, m, den, sc.x));
      if (TAIL) kahan_tail<T>(p, k);
    } else {
      p = addcdiv_op<T>(p, m, den, sc.x);  // rounded by the store
    }
  }
};

}  // namespace optimi
