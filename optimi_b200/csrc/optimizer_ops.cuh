// Per-element arithmetic of the eight optimizers, as "ops" for mta_kernel.
//
// Every op replays the reference's foreach sequence for its optimizer in registers: each line that
// ends in rnd<T>(...) is ONE ATen op of that sequence — an fp32 computation followed by a rounding
// to the storage type — in the reference's order, with the fp32 formula the CUDA build of that
// ATen op uses (fused multiply-add for `x + s*y`, correctly rounded sqrt and divide, division by
// a scalar as multiplication by its reciprocal).  Intermediates that the reference keeps in the
// gradient buffer live in registers here, so gradients are never written.
//
// Template flags: KAHAN = Kahan-compensated update (low-precision storage only), UPDATE = false is
// the optimizer-accumulation micro-step (state averages only).
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
  const float d = rnd<T>(__fsqrt_rn(v));
  return rnd<T>(__fadd_rn(d, eps));
}

// addcdiv: x + value * (a / b)
__device__ __forceinline__ float addcdiv_op(float x, float a, float b, float value) {
  return __fmaf_rn(value, __fdiv_rn(a, b), x);
}

struct Lerp {  // uniform pieces of one scalar-weight lerp
  float w, omw;
  int low;
};

// ---------------------------------------------------------------------------------------------
// Adam / AdamW                       lists: 0 p, 1 g, 2 m (exp_avg), 3 v (exp_avg_sq), 4 k (kahan)
// optimi/adam.py:424-453
// ---------------------------------------------------------------------------------------------
struct AdamArgs {
  Lerp l1;
  float beta2_hat, beta2_comp, wd, eps, neg_lr;
  int wd_mode;
};

template <typename T>
__device__ __forceinline__ void adam_moments(float& m, float& v, float g, const Lerp& l1, float beta2_hat,
                                             float beta2_comp) {
  m = rnd<T>(lerp_op(m, g, l1.w, l1.omw, l1.low));
  v = rnd<T>(__fmul_rn(v, beta2_hat));
  v = rnd<T>(__fmaf_rn(beta2_comp, __fmul_rn(g, g), v));
}

template <bool KAHAN, bool UPDATE>
struct AdamOp {
  static constexpr int NL = 5;
  using Args = AdamArgs;
  template <typename T, int N>
  static __device__ __forceinline__ void run(T* const (&ptr)[NL], int i, const Args& a) {
    float p[N], g[N], m[N], v[N], k[N];
    Pack<T, N>::load(ptr[1] + i, g);
    Pack<T, N>::load(ptr[2] + i, m);
    Pack<T, N>::load(ptr[3] + i, v);
    if (UPDATE) Pack<T, N>::load(ptr[0] + i, p);
    if (KAHAN) Pack<T, N>::load(ptr[4] + i, k);
#pragma unroll
    for (int j = 0; j < N; j++) {
      if (UPDATE) {
        if (a.wd_mode == kWdDecoupled) p[j] = rnd<T>(__fmul_rn(p[j], a.wd));
        else if (a.wd_mode == kWdL2) g[j] = rnd<T>(__fmaf_rn(a.wd, p[j], g[j]));
      }
      adam_moments<T>(m[j], v[j], g[j], a.l1, a.beta2_hat, a.beta2_comp);
      if (UPDATE) {
        const float den = denominator<T>(v[j], a.eps);
        if (KAHAN) {
          k[j] = rnd<T>(addcdiv_op(k[j], m[j], den, a.neg_lr));
          kahan_tail<T>(p[j], k[j]);
        } else {
          p[j] = rnd<T>(addcdiv_op(p[j], m[j], den, a.neg_lr));
        }
      }
    }
    Pack<T, N>::store(ptr[2] + i, m);
    Pack<T, N>::store(ptr[3] + i, v);
    if (UPDATE) Pack<T, N>::store(ptr[0] + i, p);
    if (KAHAN) Pack<T, N>::store(ptr[4] + i, k);
  }
};

// ---------------------------------------------------------------------------------------------
// RAdam and Ranger          lists: 0 p, 1 g, 2 m, 3 v, 4 k, 5 la (slow weights, Ranger only)
// optimi/radam.py:438-479, optimi/ranger.py:498-561
// ---------------------------------------------------------------------------------------------
struct RangerArgs {
  Lerp l1;
  float beta2_hat, beta2_comp, wd, eps, neg_lr;  // neg_lr = -lr*rect when use_rect
  float alpha;
  int wd_mode, use_rect, lookahead;
};

template <bool KAHAN, bool UPDATE>
struct RangerOp {
  static constexpr int NL = 6;
  using Args = RangerArgs;
  template <typename T, int N>
  static __device__ __forceinline__ void run(T* const (&ptr)[NL], int i, const Args& a) {
    float p[N], g[N], m[N], v[N], k[N], la[N];
    const bool look = UPDATE && a.lookahead;
    Pack<T, N>::load(ptr[1] + i, g);
    Pack<T, N>::load(ptr[2] + i, m);
    Pack<T, N>::load(ptr[3] + i, v);
    if (UPDATE) Pack<T, N>::load(ptr[0] + i, p);
    if (KAHAN) Pack<T, N>::load(ptr[4] + i, k);
    if (look) Pack<T, N>::load(ptr[5] + i, la);
#pragma unroll
    for (int j = 0; j < N; j++) {
      if (UPDATE) {
        if (a.wd_mode == kWdDecoupled) p[j] = rnd<T>(__fmul_rn(p[j], a.wd));
        else if (a.wd_mode == kWdL2) g[j] = rnd<T>(__fmaf_rn(a.wd, p[j], g[j]));
      }
      adam_moments<T>(m[j], v[j], g[j], a.l1, a.beta2_hat, a.beta2_comp);
      if (UPDATE) {
        float x = KAHAN ? k[j] : p[j];
        if (a.use_rect) x = rnd<T>(addcdiv_op(x, m[j], denominator<T>(v[j], a.eps), a.neg_lr));
        else x = rnd<T>(__fmaf_rn(a.neg_lr, m[j], x));
        if (KAHAN) {
          k[j] = x;
          kahan_tail<T>(p[j], k[j]);
          if (look) {  // optimi/ranger.py:537-549
            const float diff = rnd<T>(__fsub_rn(p[j], la[j]));
            k[j] = rnd<T>(__fmaf_rn(a.alpha, diff, k[j]));
            kahan_tail<T>(la[j], k[j]);
            p[j] = la[j];
          }
        } else {
          p[j] = x;
          if (look) {  // optimi/ranger.py:559-561
            p[j] = rnd<T>(__fsub_rn(p[j], la[j]));
            la[j] = rnd<T>(__fmaf_rn(a.alpha, p[j], la[j]));
            p[j] = la[j];
          }
        }
      }
    }
    Pack<T, N>::store(ptr[2] + i, m);
    Pack<T, N>::store(ptr[3] + i, v);
    if (UPDATE) Pack<T, N>::store(ptr[0] + i, p);
    if (KAHAN) Pack<T, N>::store(ptr[4] + i, k);
    if (look) Pack<T, N>::store(ptr[5] + i, la);
  }
};

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
struct LionOp {
  static constexpr int NL = 4;
  using Args = LionArgs;
  template <typename T, int N>
  static __device__ __forceinline__ void run(T* const (&ptr)[NL], int i, const Args& a) {
    float p[N], g[N], m[N], k[N];
    Pack<T, N>::load(ptr[1] + i, g);
    Pack<T, N>::load(ptr[2] + i, m);
    if (UPDATE) Pack<T, N>::load(ptr[0] + i, p);
    if (KAHAN) Pack<T, N>::load(ptr[3] + i, k);
#pragma unroll
    for (int j = 0; j < N; j++) {
      float u = 0.f;
      if (UPDATE) {
        if (a.wd_mode == kWdDecoupled) p[j] = rnd<T>(__fmul_rn(p[j], a.wd));
        u = rnd<T>(lerp_op(m[j], g[j], a.l1.w, a.l1.omw, a.l1.low));
        u = (float)((0.f < u) - (u < 0.f));
      }
      m[j] = rnd<T>(lerp_op(m[j], g[j], a.l2.w, a.l2.omw, a.l2.low));
      if (UPDATE) {
        if (KAHAN) {
          k[j] = rnd<T>(__fmaf_rn(a.neg_lr, u, k[j]));
          kahan_tail<T>(p[j], k[j]);
        } else {
          p[j] = rnd<T>(__fmaf_rn(a.neg_lr, u, p[j]));
        }
      }
    }
    Pack<T, N>::store(ptr[2] + i, m);
    if (UPDATE) Pack<T, N>::store(ptr[0] + i, p);
    if (KAHAN) Pack<T, N>::store(ptr[3] + i, k);
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
struct SgdOp {
  static constexpr int NL = 4;
  using Args = SgdArgs;
  template <typename T, int N>
  static __device__ __forceinline__ void run(T* const (&ptr)[NL], int i, const Args& a) {
    float p[N], g[N], m[N], k[N];
    Pack<T, N>::load(ptr[1] + i, g);
    if (a.has_momentum) Pack<T, N>::load(ptr[2] + i, m);
    if (UPDATE) Pack<T, N>::load(ptr[0] + i, p);
    if (KAHAN) Pack<T, N>::load(ptr[3] + i, k);
#pragma unroll
    for (int j = 0; j < N; j++) {
      if (UPDATE) {
        if (a.wd_mode == kWdDecoupled) p[j] = rnd<T>(__fmul_rn(p[j], a.wd));
        else if (a.wd_mode == kWdL2) g[j] = rnd<T>(__fmaf_rn(a.wd, p[j], g[j]));
      }
      float upd = g[j];
      if (a.has_momentum) {
        if (a.dampening) {
          m[j] = rnd<T>(lerp_op(m[j], g[j], a.damp.w, a.damp.omw, a.damp.low));
        } else {
          m[j] = rnd<T>(__fmul_rn(m[j], a.momentum));
          m[j] = rnd<T>(__fadd_rn(m[j], g[j]));
        }
        upd = m[j];
      }
      if (UPDATE) {
        if (KAHAN) {
          k[j] = rnd<T>(__fmaf_rn(a.neg_lr, upd, k[j]));
          kahan_tail<T>(p[j], k[j]);
        } else {
          p[j] = rnd<T>(__fmaf_rn(a.neg_lr, upd, p[j]));
        }
      }
    }
    if (a.has_momentum) Pack<T, N>::store(ptr[2] + i, m);
    if (UPDATE) Pack<T, N>::store(ptr[0] + i, p);
    if (KAHAN) Pack<T, N>::store(ptr[3] + i, k);
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
struct AdanOp {
  static constexpr int NL = 7;
  using Args = AdanArgs;
  template <typename T, int N>
  static __device__ __forceinline__ void run(T* const (&ptr)[NL], int i, const Args& a) {
    float p[N], g[N], m[N], d[N], q[N], pg[N], k[N];
    Pack<T, N>::load(ptr[1] + i, g);
    Pack<T, N>::load(ptr[2] + i, m);
    Pack<T, N>::load(ptr[3] + i, d);
    Pack<T, N>::load(ptr[4] + i, q);
    Pack<T, N>::load(ptr[5] + i, pg);
    if (UPDATE) Pack<T, N>::load(ptr[0] + i, p);
    if (KAHAN) Pack<T, N>::load(ptr[6] + i, k);
#pragma unroll
    for (int j = 0; j < N; j++) {
      float diff = rnd<T>(__fadd_rn(pg[j], g[j]));
      m[j] = rnd<T>(lerp_op(m[j], g[j], a.l1.w, a.l1.omw, a.l1.low));
      d[j] = rnd<T>(lerp_op(d[j], diff, a.l2.w, a.l2.omw, a.l2.low));
      diff = rnd<T>(__fmul_rn(diff, a.beta2));
      diff = rnd<T>(__fadd_rn(diff, g[j]));
      q[j] = rnd<T>(__fmul_rn(q[j], a.beta3_hat));
      q[j] = rnd<T>(__fmaf_rn(a.beta3_comp, __fmul_rn(diff, diff), q[j]));
      pg[j] = -g[j];
      if (UPDATE) {
        const float den = denominator<T>(q[j], a.eps);
        if (a.wd_mode == 1) p[j] = rnd<T>(__fmul_rn(p[j], a.wd_mul));
        if (KAHAN) {
          k[j] = rnd<T>(addcdiv_op(k[j], m[j], den, a.neg_lr));
          k[j] = rnd<T>(addcdiv_op(k[j], d[j], den, a.neg_lr_beta2));
          kahan_tail<T>(p[j], k[j]);
        } else {
          p[j] = rnd<T>(addcdiv_op(p[j], m[j], den, a.neg_lr));
          p[j] = rnd<T>(addcdiv_op(p[j], d[j], den, a.neg_lr_beta2));
        }
        if (a.wd_mode == 2) p[j] = rnd<T>(__fmul_rn(p[j], a.wd_mul));
      }
    }
    Pack<T, N>::store(ptr[2] + i, m);
    Pack<T, N>::store(ptr[3] + i, d);
    Pack<T, N>::store(ptr[4] + i, q);
    Pack<T, N>::store(ptr[5] + i, pg);
    if (UPDATE) Pack<T, N>::store(ptr[0] + i, p);
    if (KAHAN) Pack<T, N>::store(ptr[6] + i, k);
  }
};

// ---------------------------------------------------------------------------------------------
// StableAdamW, pass B (parameter update)                    lists: 0 p, 1 m, 2 v, 3 k
// optimi/stableadamw.py:522-544.  The clipped -lr and the weight-decay factor are per tensor.
// ---------------------------------------------------------------------------------------------
struct StableUpdateArgs {
  float eps;
  int has_wd;
};

template <typename T, bool KAHAN, int N>
__device__ __forceinline__ void stable_update_run(T* const (&ptr)[4], int i, const StableUpdateArgs& a, float neg_lr,
                                                  float wd) {
  float p[N], m[N], v[N], k[N];
  Pack<T, N>::load(ptr[0] + i, p);
  Pack<T, N>::load(ptr[1] + i, m);
  Pack<T, N>::load(ptr[2] + i, v);
  if (KAHAN) Pack<T, N>::load(ptr[3] + i, k);
#pragma unroll
  for (int j = 0; j < N; j++) {
    if (a.has_wd) p[j] = rnd<T>(__fmul_rn(p[j], wd));
    const float den = denominator<T>(v[j], a.eps);
    if (KAHAN) {
      k[j] = rnd<T>(addcdiv_op(k[j], m[j], den, neg_lr));
      kahan_tail<T>(p[j], k[j]);
    } else {
      p[j] = rnd<T>(addcdiv_op(p[j], m[j], den, neg_lr));
    }
  }
  Pack<T, N>::store(ptr[0] + i, p);
  if (KAHAN) Pack<T, N>::store(ptr[3] + i, k);
}

}  // namespace optimi
