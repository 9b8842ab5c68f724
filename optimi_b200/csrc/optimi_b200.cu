// C ABI of the sm_100a optimizer-step kernels: argument checking, by-value table building,
// kernel launches.  See include/optimi_b200.h for the contract of every entry point.
#include "../../include/optimi_b200.h"

#include <atomic>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <type_traits>
#include <vector>

#include "optimizer_ops.cuh"

namespace optimi {

// ---------------------------------------------------------------------------------------------
// errors
// ---------------------------------------------------------------------------------------------
// The library may be compiled as one translation unit or as several in parallel (OPTIMI_PART = 0, 1, 2:
// see optimi_b200/build.py); part 0 owns the process-wide state, the others refer to it.
#define COMMA ,
#if defined(OPTIMI_PART) && OPTIMI_PART != 0
#define OPTIMI_SHARED(decl, init) extern decl
#else
#define OPTIMI_SHARED(decl, init) decl init
#endif
#if defined(OPTIMI_PART)
#define OPTIMI_IN_PART(p) (OPTIMI_PART == (p))
#else
#define OPTIMI_IN_PART(p) 1
#endif
OPTIMI_SHARED(thread_local char g_error[512], = "");

static int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return code;
}

OPTIMI_SHARED(std::atomic<unsigned long long> g_launches, {0});

// ---------------------------------------------------------------------------------------------
// launches, and their life inside a CUDA graph
// ---------------------------------------------------------------------------------------------
// Every kernel receives its scalars by value, so a launch captured into a CUDA graph would repeat
// the scalars of the step it was captured at (bias corrections, learning rate) on every replay.
// Instead of a second family of kernels that read their scalars from device memory, the library
// remembers which graph nodes its launches became (record mode) and later rewrites those nodes'
// kernel parameters in the instantiated graph with the scalars of the coming step (update mode):
// the caller repeats the very same step calls, and each would-be launch turns into one
// cudaGraphExecKernelNodeSetParams.  Outside both modes a launch into a capturing stream is
// refused, because it would silently freeze the step count.
struct GraphNodes {
  std::vector<cudaGraphNode_t> nodes;
};
enum GraphMode : int { kGraphNone = 0, kGraphRecord = 1, kGraphUpdate = 2 };
struct GraphState {
  int mode;
  GraphNodes* nodes;      // record: being filled; update: being walked
  size_t cursor;          // update: next node
  cudaGraphExec_t exec;   // update: the instantiated graph
};
OPTIMI_SHARED(thread_local GraphState g_graph, = {kGraphNone COMMA nullptr COMMA 0 COMMA nullptr});

template <class... P>
static int launch_kernel(const char* what, void (*kernel)(P...), unsigned grid, unsigned block, cudaStream_t stream,
                         const P&... params) {
  void* kernel_params[] = {const_cast<void*>(static_cast<const void*>(&params))...};
  if (g_graph.mode == kGraphUpdate) {
    GraphNodes& gn = *g_graph.nodes;
    if (g_graph.cursor >= gn.nodes.size())
      return fail(OPTIMI_ERR_INVALID_ARGUMENT, "%s: this step issues more launches than were recorded (%zu); capture it again", what,
                  gn.nodes.size());
    cudaKernelNodeParams np;
    memset(&np, 0, sizeof(np));
    np.func = reinterpret_cast<void*>(kernel);
    np.gridDim = dim3(grid);
    np.blockDim = dim3(block);
    np.sharedMemBytes = 0;
    np.kernelParams = kernel_params;
    np.extra = nullptr;
    cudaError_t e = cudaGraphExecKernelNodeSetParams(g_graph.exec, gn.nodes[g_graph.cursor], &np);
    if (e != cudaSuccess) {
      cudaGetLastError();
      return fail(OPTIMI_ERR_CUDA, "%s: cudaGraphExecKernelNodeSetParams on recorded node %zu: %s", what, g_graph.cursor,
                  cudaGetErrorString(e));
    }
    g_graph.cursor++;
    return OPTIMI_OK;
  }
  cudaStreamCaptureStatus status = cudaStreamCaptureStatusNone;
  cudaError_t e = cudaStreamIsCapturing(stream, &status);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(OPTIMI_ERR_CUDA, "%s: cudaStreamIsCapturing: %s", what, cudaGetErrorString(e));
  }
  if (g_graph.mode == kGraphNone && status != cudaStreamCaptureStatusNone)
    return fail(OPTIMI_ERR_CAPTURE,
                "%s: the stream is capturing a CUDA graph; a plain launch would repeat this step's scalars on every replay. "
                "Bracket the step with optimi_b200_graph_record_begin/_end and refresh the graph with "
                "optimi_b200_graph_update_begin/_end before each replay",
                what);
  if (g_graph.mode == kGraphRecord && status != cudaStreamCaptureStatusActive)
    return fail(OPTIMI_ERR_CAPTURE, "%s: recording graph nodes, but the stream is not capturing", what);
  e = cudaLaunchKernel(reinterpret_cast<const void*>(kernel), dim3(grid), dim3(block), kernel_params, 0, stream);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(OPTIMI_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
  }
  if (g_graph.mode == kGraphRecord) {
    // the node this launch became is the stream's only capture dependency now
    const cudaGraphNode_t* deps = nullptr;
    size_t n_deps = 0;
    e = cudaStreamGetCaptureInfo(stream, &status, nullptr, nullptr, &deps, &n_deps);
    if (e != cudaSuccess || status != cudaStreamCaptureStatusActive || n_deps != 1 || !deps) {
      cudaGetLastError();
      return fail(OPTIMI_ERR_CUDA, "%s: cannot identify the captured kernel node (%s, %zu dependencies)", what,
                  cudaGetErrorString(e), n_deps);
    }
    g_graph.nodes->nodes.push_back(deps[0]);
  }
  return OPTIMI_OK;
}

static Lerp make_lerp(double weight) {
  const float w = (float)weight;
  Lerp l;
  l.low = fabsf(w) < 0.5f;
  l.x = l.low ? w : -(1.0f - w);
  return l;
}

static int check_lists(const char* name, int n, const int64_t* numels, int dtype, int n_lists, void* const* const* lists,
                       const bool* required, const char* const* list_names) {
  if (n < 0) return fail(OPTIMI_ERR_INVALID_ARGUMENT, "%s: n_tensors=%d is negative", name, n);
  if (dtype != OPTIMI_F32 && dtype != OPTIMI_BF16 && dtype != OPTIMI_F16)
    return fail(OPTIMI_ERR_INVALID_ARGUMENT, "%s: unknown dtype code %d", name, dtype);
  if (n == 0) return OPTIMI_OK;
  if (!numels) return fail(OPTIMI_ERR_INVALID_ARGUMENT, "%s: numels is NULL", name);
  for (int l = 0; l < n_lists; l++) {
    if (required[l] && !lists[l]) return fail(OPTIMI_ERR_INVALID_ARGUMENT, "%s: list `%s` is NULL", name, list_names[l]);
  }
  for (int i = 0; i < n; i++) {
    if (numels[i] < 0) return fail(OPTIMI_ERR_INVALID_ARGUMENT, "%s: numels[%d]=%lld is negative", name, i, (long long)numels[i]);
    if (numels[i] == 0) continue;
    for (int l = 0; l < n_lists; l++) {
      if (required[l] && !lists[l][i])
        return fail(OPTIMI_ERR_INVALID_ARGUMENT, "%s: `%s`[%d] is a NULL pointer for a tensor of %lld elements", name,
                    list_names[l], i, (long long)numels[i]);
    }
  }
  return OPTIMI_OK;
}

// Walks the tensor list, filling one by-value table after another and handing each to `launch`.
// `tile` = elements per block.
template <int NL, bool SMALL, class Launch>
static int for_each_table(int n, const int64_t* numels, void* const* const (&lists)[NL], int tile, Launch&& launch) {
  using Table = MtaTable<NL, SMALL>;
  Table tab;  // ~30 KB on the host stack
  int i = 0, tile_base = 0;
  while (i < n) {
    int count = 0, tiles = 0;
    tab.tensor_base = i;
    tab.tile_base = tile_base;
    while (i < n && count < Table::CAP) {
      const long long c = (numels[i] + tile - 1) / tile;
      if ((long long)tiles + c > 0x7fffffffLL - 1) break;
      for (int l = 0; l < NL; l++) tab.ptr[l][count] = lists[l] ? lists[l][i] : nullptr;
      tab.numel[count] = numels[i];
      tab.tile_start[count] = tiles;
      tiles += (int)c;
      count++;
      i++;
    }
    if (count == 0) return fail(OPTIMI_ERR_INVALID_ARGUMENT, "tensor %d has too many elements for one launch", i);
    tab.tile_start[count] = tiles;
    tab.n_tensors = count;
    // coarse index: bucket b covers blocks [b << shift, (b+1) << shift)
    int shift = 0;
    while ((tiles >> shift) >= Table::NB) shift++;
    tab.bucket_shift = shift;
    for (int b = 0, t = 0; b < Table::NB; b++) {
      const long long first = (long long)b << shift;
      while (t + 1 < count && tab.tile_start[t + 1] <= first) t++;
      tab.bucket_tensor[b] = t;
    }
    if (tiles > 0) {
      int rc = launch(tab, tiles);
      if (rc != OPTIMI_OK) return rc;
    }
    tile_base += tiles;
  }
  return OPTIMI_OK;
}

// elements one block covers
template <typename T, class Op>
constexpr int tile_of() { return kThreads * Op::U * VecN<T>::N; }

template <typename T, class Op>
static int launch_op(const char* name, int n, const int64_t* numels, void* const* const (&lists)[Op::NL],
                     const typename Op::Args& args, cudaStream_t stream) {
  if (n <= MtaTable<Op::NL, true>::CAP) {  // few tensors (a gradient-release step): the small table
    return for_each_table<Op::NL, true>(n, numels, lists, tile_of<T, Op>(), [&](const MtaTable<Op::NL, true>& tab, int tiles) {
      return launch_kernel(name, mta_kernel<T, Op, true>, tiles, kThreads, stream, tab, args);
    });
  }
  return for_each_table<Op::NL, false>(n, numels, lists, tile_of<T, Op>(), [&](const MtaTable<Op::NL, false>& tab, int tiles) {
    return launch_kernel(name, mta_kernel<T, Op, false>, tiles, kThreads, stream, tab, args);
  });
}

// Gradient factor requested for the calling thread's next launches (optimi_b200_grad_scale_begin / _end).
OPTIMI_SHARED(thread_local const float* g_grad_factor, = nullptr);

// Launches Op, or ScaledOp<Op> when a gradient factor is active.
template <typename T, class Op>
static int launch_maybe_scaled(const char* name, int n, const int64_t* numels, void* const* const (&lists)[Op::NL],
                               const typename Op::Args& args, cudaStream_t stream) {
  if (g_grad_factor) {
    ScaledArgs<typename Op::Args> sa;
    sa.base = args;
    sa.factor = g_grad_factor;
    return launch_op<T, ScaledOp<Op>>(name, n, numels, lists, sa, stream);
  }
  return launch_op<T, Op>(name, n, numels, lists, args, stream);
}

// Peer push / pull requested for the calling thread's next launches (optimi_b200_push_begin,
// optimi_b200_pull_begin and their _end).
OPTIMI_SHARED(thread_local PeerPush g_push, = {0 COMMA {0}});
OPTIMI_SHARED(thread_local PeerPull g_pull, = {0 COMMA 1.0f COMMA {0}});

// Launches Op, or PeerOp<Op, ...> when a peer push and/or pull is active.  PULLABLE is false for the
// ops without a gradient list at position 1 (StableAdamW's passes).
template <typename T, class Op, bool PULLABLE = true>
static int launch_maybe_push(const char* name, int n, const int64_t* numels, void* const* const (&lists)[Op::NL],
                             const typename Op::Args& args, cudaStream_t stream) {
  if (g_pull.n > 0) {
    if (g_grad_factor)
      return fail(OPTIMI_ERR_INVALID_ARGUMENT, "%s: a gradient factor cannot be combined with the gradient pull", name);
    if constexpr (PULLABLE) {
      PeerArgs<typename Op::Args> pa;
      pa.base = args;
      pa.push = g_push;
      pa.pull = g_pull;
      if (g_pull.n <= 2) return launch_op<T, PeerOp<Op, 2>>(name, n, numels, lists, pa, stream);
      if (g_pull.n <= 4) return launch_op<T, PeerOp<Op, 4>>(name, n, numels, lists, pa, stream);
      return launch_op<T, PeerOp<Op, 8>>(name, n, numels, lists, pa, stream);
    } else {
      return fail(OPTIMI_ERR_INVALID_ARGUMENT, "%s: the gradient pull is not available for this optimizer", name);
    }
  }
  if (g_push.n > 0) {
    if constexpr (PULLABLE) {
      if (g_grad_factor) {  // scale the gradients on load, push the parameters on store
        PeerArgs<ScaledArgs<typename Op::Args>> pa;
        pa.base.base = args;
        pa.base.factor = g_grad_factor;
        pa.push = g_push;
        pa.pull.n = 0;
        return launch_op<T, PeerOp<ScaledOp<Op>, 0>>(name, n, numels, lists, pa, stream);
      }
    }
    PeerArgs<typename Op::Args> pa;
    pa.base = args;
    pa.push = g_push;
    pa.pull.n = 0;
    return launch_op<T, PeerOp<Op, 0>>(name, n, numels, lists, pa, stream);
  }
  if constexpr (PULLABLE) {  // the ops with a gradient list
    return launch_maybe_scaled<T, Op>(name, n, numels, lists, args, stream);
  } else {
    return launch_op<T, Op>(name, n, numels, lists, args, stream);
  }
}

// Picks the instantiation for (dtype, kahan, update).  Kahan compensation exists only for the
// 16-bit storage types, as in the reference (e.g. optimi/adam.py:421).
template <template <bool, bool> class Op, class Lists, class Args>
static int dispatch(const char* name, int dtype, bool kahan, bool update, int n, const int64_t* numels, const Lists& lists,
                    const Args& args, cudaStream_t stream) {
#define OPTIMI_GO(T)                                                                                   \
  do {                                                                                                 \
    if (!update) return launch_maybe_scaled<T, Op<false, false>>(name, n, numels, lists, args, stream); \
    if (kahan) return launch_maybe_push<T, Op<true, true>>(name, n, numels, lists, args, stream);      \
    return launch_maybe_push<T, Op<false, true>>(name, n, numels, lists, args, stream);                \
  } while (0)
  switch (dtype) {
    case OPTIMI_F32:
      if (!update) return launch_maybe_scaled<float, Op<false, false>>(name, n, numels, lists, args, stream);
      return launch_maybe_push<float, Op<false, true>>(name, n, numels, lists, args, stream);
    case OPTIMI_BF16: OPTIMI_GO(__nv_bfloat16);
    case OPTIMI_F16: OPTIMI_GO(__half);
  }
#undef OPTIMI_GO
  return fail(OPTIMI_ERR_INVALID_ARGUMENT, "%s: unknown dtype code %d", name, dtype);
}

// ---------------------------------------------------------------------------------------------
// StableAdamW kernels
// ---------------------------------------------------------------------------------------------
// Pass A with the per-tile sum: advances both averages and writes the tile's sum of
// g^2 / max(v, eps^2) to partial[tile] — one double per tile, written (not accumulated), so the
// scratch needs no clearing and the result does not depend on block scheduling.
// Op = StableMomentsOp<true> (or its ScaledOp) for StableAdamW, SumSqOp for the gradient norm.
template <typename T, class Op, bool SMALL>
__global__ void __launch_bounds__(kThreads, kStableMinBlocks) tile_sum_kernel(const __grid_constant__ MtaTable<Op::NL, SMALL> tab,
                                                                             const __grid_constant__ typename Op::Args a,
                                                                             double* __restrict__ partial) {
  Span s;
  double acc = process_tile<T, Op>(tab, a, s);
  __shared__ double warp_sum[kThreads / 32];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_down_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) warp_sum[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    double t = 0.0;
#pragma unroll
    for (int w = 0; w < kThreads / 32; w++) t += warp_sum[w];
    partial[tab.tile_base + blockIdx.x] = t;
  }
}

struct StableFinalizeArgs {
  double lr, weight_decay, max_lr;
  int decouple_lr;
};

// One block per tensor: folds the tensor's tile partials in a fixed order, then does on the device
// what the reference does on the host after `.item()` (optimi/stableadamw.py:512-524): mean and
// square root rounded to the storage type, -lr / max(1, rms) and the weight-decay factor in double.
template <typename T, bool SMALL>
__global__ void __launch_bounds__(256) stable_finalize_kernel(const __grid_constant__ MtaTable<4, SMALL> tab,
                                                              const __grid_constant__ StableFinalizeArgs a,
                                                              const double* __restrict__ partial,
                                                              float2* __restrict__ tensor_scalars) {
  const int t = blockIdx.x;
  const int c0 = tab.tile_start[t], c1 = tab.tile_start[t + 1];
  double acc = 0.0;
  for (int c = c0 + threadIdx.x; c < c1; c += 256) acc += partial[tab.tile_base + c];
  __shared__ double warp_sum[8];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_down_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) warp_sum[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    double sum = 0.0;
    for (int w = 0; w < 8; w++) sum += warp_sum[w];
    const long long n = tab.numel[t];
    float2 out = make_float2((float)(-a.lr), 1.0f);
    if (n > 0) {
      const float mean = rnd<T>((float)(sum / (double)n));
      const float rms = rnd<T>(__fsqrt_rn(mean));
      const double neg_lr = -a.lr / fmax(1.0, (double)rms);
      const double wd = a.decouple_lr ? 1.0 + (neg_lr / a.max_lr) * a.weight_decay : 1.0 + neg_lr * a.weight_decay;
      out = make_float2((float)neg_lr, (float)wd);
    }
    tensor_scalars[tab.tensor_base + t] = out;
  }
}

// ---------------------------------------------------------------------------------------------
// Gradient-norm clip factor: what torch.nn.utils.clip_grad_norm_ computes before it scales the
// gradients (torch/nn/utils/clip_grad.py): per-tensor 2-norms in the storage type, the 2-norm of
// those, and min(1, max_norm * (1 / (total + 1e-6))) with every intermediate rounded to the storage
// type.  Pass 1 is tile_sum_kernel<T, SumSqOp>; these two finish the job.
// ---------------------------------------------------------------------------------------------
template <typename T, bool SMALL>
__global__ void __launch_bounds__(256) norm_finalize_kernel(const __grid_constant__ MtaTable<2, SMALL> tab,
                                                            const double* __restrict__ partial, float* __restrict__ tensor_norms) {
  const int t = blockIdx.x;
  const int c0 = tab.tile_start[t], c1 = tab.tile_start[t + 1];
  double acc = 0.0;
  for (int c = c0 + threadIdx.x; c < c1; c += 256) acc += partial[tab.tile_base + c];
  __shared__ double warp_sum[8];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_down_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) warp_sum[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    double sum = 0.0;
    for (int w = 0; w < 8; w++) sum += warp_sum[w];
    tensor_norms[tab.tensor_base + t] = rnd<T>(__fsqrt_rn((float)sum));
  }
}

template <typename T>
__global__ void __launch_bounds__(256) clip_factor_kernel(const float* __restrict__ tensor_norms, int n_tensors, float max_norm,
                                                          float* __restrict__ out) {
  double acc = 0.0;
  for (int i = threadIdx.x; i < n_tensors; i += 256) acc += (double)tensor_norms[i] * (double)tensor_norms[i];
  __shared__ double warp_sum[8];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_down_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) warp_sum[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    double sum = 0.0;
    for (int w = 0; w < 8; w++) sum += warp_sum[w];
    const float total = rnd<T>(__fsqrt_rn((float)sum));
    const float denom = rnd<T>(__fadd_rn(total, 1e-6f));
    const float recip = rnd<T>(__fdiv_rn(1.0f, denom));
    float factor = rnd<T>(__fmul_rn(recip, max_norm));
    if (factor > 1.0f) factor = 1.0f;  // a NaN stays a NaN, as with torch.clamp
    out[0] = factor;
    out[1] = total;
  }
}

// The same clip factor in three separable steps, for gradients whose tensors are spread over several
// ranks or dtypes: per-tensor (or per-piece) sums of squares in double, to be added up by the caller
// wherever the pieces of a tensor live; per-tensor norms rounded to each tensor's storage type; the
// factor from the norms, in the storage type torch would promote the norms to.
template <bool SMALL>
__global__ void __launch_bounds__(256) sumsq_finalize_kernel(const __grid_constant__ MtaTable<2, SMALL> tab,
                                                             const double* __restrict__ partial, double* __restrict__ sumsq) {
  const int t = blockIdx.x;
  const int c0 = tab.tile_start[t], c1 = tab.tile_start[t + 1];
  double acc = 0.0;
  for (int c = c0 + threadIdx.x; c < c1; c += 256) acc += partial[tab.tile_base + c];
  __shared__ double warp_sum[8];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_down_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) warp_sum[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    double sum = 0.0;
    for (int w = 0; w < 8; w++) sum += warp_sum[w];
    sumsq[tab.tensor_base + t] = sum;
  }
}

template <typename T>
__global__ void __launch_bounds__(256) norms_from_sumsq_kernel(const double* __restrict__ sumsq, int n, float* __restrict__ norms) {
  const int i = blockIdx.x * 256 + threadIdx.x;
  if (i < n) norms[i] = rnd<T>(__fsqrt_rn((float)sumsq[i]));
}

static size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

static long long count_tiles(int n, const int64_t* numels, int tile) {
  long long c = 0;
  for (int i = 0; i < n; i++) c += (numels[i] + tile - 1) / tile;
  return c;
}

template <typename T>
static float round_to_storage(double x);
template <> float round_to_storage<float>(double x) { return (float)x; }
template <> float round_to_storage<__nv_bfloat16>(double x) { return __bfloat162float(__float2bfloat16_rn((float)x)); }
template <> float round_to_storage<__half>(double x) { return __half2float(__float2half_rn((float)x)); }

template <typename T>
static int stableadamw_typed(int n, void* const* params, void* const* grads, void* const* exp_avgs, void* const* exp_avg_sqs,
                             void* const* kahan_comps, const int64_t* numels, double lr, double beta1_comp, double beta2_hat,
                             double beta2_comp, double weight_decay, double eps, int decouple_lr, double max_lr, bool kahan,
                             bool update, void* workspace, size_t workspace_bytes, cudaStream_t stream) {
  StableMomentsArgs ma;
  ma.l1 = make_lerp(beta1_comp);
  ma.beta2_hat = (float)beta2_hat;
  ma.beta2_comp = (float)beta2_comp;
  // the reference keeps eps^2 as a 0-dim tensor of the storage type (optimi/stableadamw.py:119)
  ma.eps_sq = round_to_storage<T>(eps * eps);

  void* const* const lists_a[4] = {grads, exp_avgs, exp_avg_sqs, nullptr};
  if (!update) return launch_maybe_scaled<T, StableMomentsOp<false>>("optimi_b200_stableadamw (moments)", n, numels, lists_a, ma, stream);

  constexpr int tile_a = tile_of<T, StableMomentsOp<true>>();
  const size_t scal_bytes = align_up((size_t)n * sizeof(float2), 16);
  const size_t need = scal_bytes + (size_t)count_tiles(n, numels, tile_a) * sizeof(double);
  if (!workspace || workspace_bytes < need)
    return fail(OPTIMI_ERR_WORKSPACE_TOO_SMALL, "optimi_b200_stableadamw: workspace of %zu bytes given, %zu needed",
                workspace ? workspace_bytes : (size_t)0, need);
  if (reinterpret_cast<uintptr_t>(workspace) & 15)
    return fail(OPTIMI_ERR_INVALID_ARGUMENT, "optimi_b200_stableadamw: workspace is not 16-byte aligned");
  float2* tensor_scalars = reinterpret_cast<float2*>(workspace);
  double* partial = reinterpret_cast<double*>(reinterpret_cast<char*>(workspace) + scal_bytes);

  StableFinalizeArgs fa;
  fa.lr = lr;
  fa.weight_decay = weight_decay;
  fa.max_lr = max_lr;
  fa.decouple_lr = decouple_lr;

  auto pass_a = [&](auto small) {
    constexpr bool SMALL = decltype(small)::value;
    return for_each_table<4, SMALL>(n, numels, lists_a, tile_a, [&](const MtaTable<4, SMALL>& tab, int tiles) {
      int r;
      if (g_grad_factor) {
        ScaledArgs<StableMomentsArgs> sa;
        sa.base = ma;
        sa.factor = g_grad_factor;
        r = launch_kernel("optimi_b200_stableadamw (moments)", tile_sum_kernel<T, ScaledOp<StableMomentsOp<true>>, SMALL>, tiles,
                          kThreads, stream, tab, sa, partial);
      } else {
        r = launch_kernel("optimi_b200_stableadamw (moments)", tile_sum_kernel<T, StableMomentsOp<true>, SMALL>, tiles, kThreads,
                          stream, tab, ma, partial);
      }
      if (r != OPTIMI_OK) return r;
      const double* partial_in = partial;
      return launch_kernel("optimi_b200_stableadamw (finalize)", stable_finalize_kernel<T, SMALL>, tab.n_tensors, 256, stream,
                           tab, fa, partial_in, tensor_scalars);
    });
  };
  int rc = n <= MtaTable<4, true>::CAP ? pass_a(std::true_type{}) : pass_a(std::false_type{});
  if (rc != OPTIMI_OK) return rc;

  StableUpdateArgs ua;
  ua.tensor_scalars = tensor_scalars;
  ua.eps = (float)eps;
  ua.has_wd = weight_decay != 0;
  void* const* const lists_b[4] = {params, exp_avgs, exp_avg_sqs, kahan ? kahan_comps : nullptr};
  if constexpr (sizeof(T) == 2) {  // Kahan compensation exists for the 16-bit storage types only
    if (kahan) return launch_maybe_push<T, StableUpdateOp<true>, false>("optimi_b200_stableadamw (update)", n, numels, lists_b, ua, stream);
  }
  return launch_maybe_push<T, StableUpdateOp<false>, false>("optimi_b200_stableadamw (update)", n, numels, lists_b, ua, stream);
}

static int wd_mode_of(double weight_decay, int decouple_wd) {
  if (weight_decay == 0) return kWdNone;
  return decouple_wd ? kWdDecoupled : kWdL2;
}

static bool low_precision(int dtype) { return dtype == OPTIMI_BF16 || dtype == OPTIMI_F16; }

}  // namespace optimi

using namespace optimi;

extern "C" {

#if OPTIMI_IN_PART(0)
const char* optimi_b200_last_error(void) { return g_error; }

int optimi_b200_version(void) { return 100; }

int optimi_b200_push_begin(int n_peers, const int64_t* peer_deltas) {
  const char* fn = "optimi_b200_push_begin";
  if (n_peers < 0 || n_peers > kMaxPeers) return fail(OPTIMI_ERR_INVALID_ARGUMENT, "%s: n_peers=%d is outside 0..%d", fn, n_peers, kMaxPeers);
  if (n_peers > 0 && !peer_deltas) return fail(OPTIMI_ERR_INVALID_ARGUMENT, "%s: peer_deltas is NULL", fn);
  for (int j = 0; j < n_peers; j++)
    if (peer_deltas[j] % 16) return fail(OPTIMI_ERR_INVALID_ARGUMENT, "%s: peer_deltas[%d] is not a multiple of 16 bytes", fn, j);
  g_push.n = n_peers;
  for (int j = 0; j < kMaxPeers; j++) g_push.delta[j] = j < n_peers ? (long long)peer_deltas[j] : 0;
  return OPTIMI_OK;
}

void optimi_b200_push_end(void) { g_push.n = 0; }

int optimi_b200_pull_begin(int n_ranks, const int64_t* grad_deltas, double scale) {
  const char* fn = "optimi_b200_pull_begin";
  if (n_ranks < 0 || n_ranks > kMaxRanks) return fail(OPTIMI_ERR_INVALID_ARGUMENT, "%s: n_ranks=%d is outside 0..%d", fn, n_ranks, kMaxRanks);
  if (n_ranks > 0 && !grad_deltas) return fail(OPTIMI_ERR_INVALID_ARGUMENT, "%s: grad_deltas is NULL", fn);
  for (int r = 0; r < n_ranks; r++)
    if (grad_deltas[r] % 16) return fail(OPTIMI_ERR_INVALID_ARGUMENT, "%s: grad_deltas[%d] is not a multiple of 16 bytes", fn, r);
  g_pull.n = n_ranks;
  g_pull.scale = (float)scale;
  for (int r = 0; r < kMaxRanks; r++) g_pull.delta[r] = r < n_ranks ? (long long)grad_deltas[r] : 0;
  return OPTIMI_OK;
}

void optimi_b200_pull_end(void) { g_pull.n = 0; }

unsigned long long optimi_b200_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int optimi_b200_graph_record_begin(void) {
  if (g_graph.mode != kGraphNone)
    return fail(OPTIMI_ERR_INVALID_ARGUMENT, "optimi_b200_graph_record_begin: a record or update bracket is already open on this thread");
  g_graph.mode = kGraphRecord;
  g_graph.nodes = new GraphNodes();
  g_graph.cursor = 0;
  g_graph.exec = nullptr;
  return OPTIMI_OK;
}

int optimi_b200_graph_record_end(optimi_b200_graph_nodes** out) {
  if (g_graph.mode != kGraphRecord)
    return fail(OPTIMI_ERR_INVALID_ARGUMENT, "optimi_b200_graph_record_end: no record bracket is open on this thread");
  GraphNodes* nodes = g_graph.nodes;
  g_graph = GraphState{kGraphNone, nullptr, 0, nullptr};
  if (!out) {
    delete nodes;
    return fail(OPTIMI_ERR_INVALID_ARGUMENT, "optimi_b200_graph_record_end: out is NULL");
  }
  *out = reinterpret_cast<optimi_b200_graph_nodes*>(nodes);
  return OPTIMI_OK;
}

int optimi_b200_graph_nodes_count(const optimi_b200_graph_nodes* nodes) {
  return nodes ? (int)reinterpret_cast<const GraphNodes*>(nodes)->nodes.size() : 0;
}

void optimi_b200_graph_nodes_free(optimi_b200_graph_nodes* nodes) { delete reinterpret_cast<GraphNodes*>(nodes); }

int optimi_b200_graph_update_begin(optimi_b200_graph_nodes* nodes, void* graph_exec) {
  const char* fn = "optimi_b200_graph_update_begin";
  if (g_graph.mode != kGraphNone) return fail(OPTIMI_ERR_INVALID_ARGUMENT, "%s: a record or update bracket is already open on this thread", fn);
  if (!nodes) return fail(OPTIMI_ERR_INVALID_ARGUMENT, "%s: nodes is NULL", fn);
  if (!graph_exec) return fail(OPTIMI_ERR_INVALID_ARGUMENT, "%s: graph_exec is NULL", fn);
  g_graph.mode = kGraphUpdate;
  g_graph.nodes = reinterpret_cast<GraphNodes*>(nodes);
  g_graph.cursor = 0;
  g_graph.exec = reinterpret_cast<cudaGraphExec_t>(graph_exec);
  return OPTIMI_OK;
}

int optimi_b200_graph_update_end(void) {
  if (g_graph.mode != kGraphUpdate)
    return fail(OPTIMI_ERR_INVALID_ARGUMENT, "optimi_b200_graph_update_end: no update bracket is open on this thread");
  const size_t visited = g_graph.cursor, recorded = g_graph.nodes->nodes.size();
  g_graph = GraphState{kGraphNone, nullptr, 0, nullptr};
  if (visited != recorded)
    return fail(OPTIMI_ERR_INVALID_ARGUMENT,
                "optimi_b200_graph_update_end: the step issued %zu launches but %zu were recorded; the rest of the graph still "
                "holds the previous step's scalars — capture the step again",
                visited, recorded);
  return OPTIMI_OK;
}

int optimi_b200_adam(int n, void* const* params, void* const* grads, void* const* exp_avgs, void* const* exp_avg_sqs,
                     void* const* kahan_comps, const int64_t* numels, int dtype, double lr, double beta1_comp,
                     double beta2_hat, double beta2_comp, double weight_decay, double eps, int decouple_wd, int kahan_sum,
                     int update_parameters, void* stream) {
  const bool update = update_parameters != 0;
  const bool kahan = update && kahan_sum && kahan_comps && low_precision(dtype);
  void* const* const lists[5] = {params, grads, exp_avgs, exp_avg_sqs, kahan ? kahan_comps : nullptr};
  const bool req[5] = {update, true, true, true, kahan};
  static const char* const names[5] = {"params", "grads", "exp_avgs", "exp_avg_sqs", "kahan_comps"};
  int rc = check_lists("optimi_b200_adam", n, numels, dtype, 5, lists, req, names);
  if (rc != OPTIMI_OK || n == 0) return rc;
  AdamArgs a;
  a.l1 = make_lerp(beta1_comp);
  a.beta2_hat = (float)beta2_hat;
  a.beta2_comp = (float)beta2_comp;
  a.wd = weight_decay == 0 ? 1.0f : (float)weight_decay;  // the decay factor (or L2 coefficient); 1 = none
  a.eps = (float)eps;
  a.neg_lr = (float)(-lr);
  a.wd_mode = wd_mode_of(weight_decay, decouple_wd);
  return dispatch<AdamOp>("optimi_b200_adam", dtype, kahan, update, n, numels, lists, a, (cudaStream_t)stream);
}

#endif  // part 0 (continues below with lion and sgd)

#if OPTIMI_IN_PART(1)
int optimi_b200_radam(int n, void* const* params, void* const* grads, void* const* exp_avgs, void* const* exp_avg_sqs,
                      void* const* kahan_comps, const int64_t* numels, int dtype, double lr, double beta1_comp,
                      double beta2_hat, double beta2_comp, double weight_decay, double eps, int use_rect, double rect,
                      int decouple_wd, int kahan_sum, int update_parameters, void* stream) {
  return optimi_b200_ranger(n, params, grads, exp_avgs, exp_avg_sqs, nullptr, kahan_comps, numels, dtype, lr, beta1_comp,
                            beta2_hat, beta2_comp, weight_decay, eps, use_rect, rect, 0, 0.0, decouple_wd, kahan_sum,
                            update_parameters, stream);
}

int optimi_b200_ranger(int n, void* const* params, void* const* grads, void* const* exp_avgs, void* const* exp_avg_sqs,
                       void* const* la_params, void* const* kahan_comps, const int64_t* numels, int dtype, double lr,
                       double beta1_comp, double beta2_hat, double beta2_comp, double weight_decay, double eps, int use_rect,
                       double rect, int do_lookahead, double alpha, int decouple_wd, int kahan_sum, int update_parameters,
                       void* stream) {
  const bool update = update_parameters != 0;
  const bool kahan = update && kahan_sum && kahan_comps && low_precision(dtype);
  const bool look = update && do_lookahead;
  void* const* const lists[6] = {params, grads, exp_avgs, exp_avg_sqs, kahan ? kahan_comps : nullptr,
                                 look ? la_params : nullptr};
  const bool req[6] = {update, true, true, true, kahan, look};
  static const char* const names[6] = {"params", "grads", "exp_avgs", "exp_avg_sqs", "kahan_comps", "la_params"};
  const char* fn = la_params ? "optimi_b200_ranger" : "optimi_b200_radam";
  int rc = check_lists(fn, n, numels, dtype, 6, lists, req, names);
  if (rc != OPTIMI_OK || n == 0) return rc;
  RangerArgs a;
  a.l1 = make_lerp(beta1_comp);
  a.beta2_hat = (float)beta2_hat;
  a.beta2_comp = (float)beta2_comp;
  a.wd = weight_decay == 0 ? 1.0f : (float)weight_decay;  // the decay factor (or L2 coefficient); 1 = none
  a.eps = (float)eps;
  a.neg_lr = use_rect ? (float)(-lr * rect) : (float)(-lr);
  a.alpha = (float)alpha;
  a.wd_mode = wd_mode_of(weight_decay, decouple_wd);
  a.use_rect = use_rect != 0;
  a.lookahead = look;
  if (look) return dispatch<RangerLookOp>(fn, dtype, kahan, update, n, numels, lists, a, (cudaStream_t)stream);
  return dispatch<RadamOp>(fn, dtype, kahan, update, n, numels, lists, a, (cudaStream_t)stream);
}

#endif  // part 1 (continues below with adan)

#if OPTIMI_IN_PART(0)
int optimi_b200_lion(int n, void* const* params, void* const* grads, void* const* exp_avgs, void* const* kahan_comps,
                     const int64_t* numels, int dtype, double lr, double beta1_comp, double beta2_comp, double weight_decay,
                     int kahan_sum, int update_parameters, void* stream) {
  const bool update = update_parameters != 0;
  const bool kahan = update && kahan_sum && kahan_comps && low_precision(dtype);
  void* const* const lists[4] = {params, grads, exp_avgs, kahan ? kahan_comps : nullptr};
  const bool req[4] = {update, true, true, kahan};
  static const char* const names[4] = {"params", "grads", "exp_avgs", "kahan_comps"};
  int rc = check_lists("optimi_b200_lion", n, numels, dtype, 4, lists, req, names);
  if (rc != OPTIMI_OK || n == 0) return rc;
  LionArgs a;
  a.l1 = make_lerp(beta1_comp);
  a.l2 = make_lerp(beta2_comp);
  a.wd = weight_decay == 0 ? 1.0f : (float)weight_decay;  // the decay factor (or L2 coefficient); 1 = none
  a.neg_lr = (float)(-lr);
  a.wd_mode = weight_decay != 0 ? kWdDecoupled : kWdNone;
  return dispatch<LionOp>("optimi_b200_lion", dtype, kahan, update, n, numels, lists, a, (cudaStream_t)stream);
}

int optimi_b200_sgd(int n, void* const* params, void* const* grads, void* const* exp_avgs, void* const* kahan_comps,
                    const int64_t* numels, int dtype, double lr, double momentum, double weight_decay, int dampening,
                    int decouple_wd, int kahan_sum, int update_parameters, void* stream) {
  const bool update = update_parameters != 0;
  const bool kahan = update && kahan_sum && kahan_comps && low_precision(dtype);
  const bool has_m = momentum != 0;
  if (!has_m && !update) return OPTIMI_OK;  // nothing to accumulate into (optimi/sgd.py:352-360)
  void* const* const lists[4] = {params, grads, has_m ? exp_avgs : nullptr, kahan ? kahan_comps : nullptr};
  const bool req[4] = {update, true, has_m, kahan};
  static const char* const names[4] = {"params", "grads", "exp_avgs", "kahan_comps"};
  int rc = check_lists("optimi_b200_sgd", n, numels, dtype, 4, lists, req, names);
  if (rc != OPTIMI_OK || n == 0) return rc;
  SgdArgs a;
  a.damp = make_lerp(1 - momentum);
  a.momentum = (float)momentum;
  a.wd = weight_decay == 0 ? 1.0f : (float)weight_decay;  // the decay factor (or L2 coefficient); 1 = none
  a.neg_lr = (float)(-lr);
  a.wd_mode = wd_mode_of(weight_decay, decouple_wd);
  a.has_momentum = has_m;
  a.dampening = dampening != 0;
  return dispatch<SgdOp>("optimi_b200_sgd", dtype, kahan, update, n, numels, lists, a, (cudaStream_t)stream);
}

#endif  // part 0

#if OPTIMI_IN_PART(1)
int optimi_b200_adan(int n, void* const* params, void* const* grads, void* const* exp_avgs, void* const* exp_avg_diffs,
                     void* const* exp_avg_sqs, void* const* prev_grads, void* const* kahan_comps, const int64_t* numels,
                     int dtype, double lr, double beta1_comp, double beta2, double beta2_comp, double beta3_hat,
                     double beta3_comp, double eps, double weight_decay, int adam_wd, int kahan_sum, int update_parameters,
                     void* stream) {
  const bool update = update_parameters != 0;
  const bool kahan = update && kahan_sum && kahan_comps && low_precision(dtype);
  void* const* const lists[7] = {params, grads, exp_avgs, exp_avg_diffs, exp_avg_sqs, prev_grads, kahan ? kahan_comps : nullptr};
  const bool req[7] = {update, true, true, true, true, true, kahan};
  static const char* const names[7] = {"params", "grads", "exp_avgs", "exp_avg_diffs", "exp_avg_sqs", "prev_grads", "kahan_comps"};
  int rc = check_lists("optimi_b200_adan", n, numels, dtype, 7, lists, req, names);
  if (rc != OPTIMI_OK || n == 0) return rc;
  AdanArgs a;
  a.l1 = make_lerp(beta1_comp);
  a.l2 = make_lerp(beta2_comp);
  a.beta2 = (float)beta2;
  a.beta3_hat = (float)beta3_hat;
  a.beta3_comp = (float)beta3_comp;
  a.eps = (float)eps;
  a.neg_lr = (float)(-lr);
  a.neg_lr_beta2 = (float)(-lr * beta2);
  a.wd_mode = weight_decay == 0 ? 0 : (adam_wd ? 1 : 2);
  // Adan-style decay divides by the factor; the reference's CUDA op multiplies by the reciprocal,
  // taken in double precision and then narrowed to fp32
  a.wd_mul = weight_decay == 0 ? 1.0f : (adam_wd ? (float)weight_decay : (float)(1.0 / weight_decay));
  return dispatch<AdanOp>("optimi_b200_adan", dtype, kahan, update, n, numels, lists, a, (cudaStream_t)stream);
}

#endif  // part 1

#if OPTIMI_IN_PART(2)
size_t optimi_b200_stableadamw_workspace_bytes(int n, const int64_t* numels) {
  if (n <= 0 || !numels) return 16;
  // the float32 tile is the smallest, so this bounds every storage type
  constexpr int tile = tile_of<float, StableMomentsOp<true>>();
  return align_up((size_t)n * sizeof(float2), 16) + (size_t)count_tiles(n, numels, tile) * sizeof(double) + 16;
}

int optimi_b200_stableadamw(int n, void* const* params, void* const* grads, void* const* exp_avgs, void* const* exp_avg_sqs,
                            void* const* kahan_comps, const int64_t* numels, int dtype, double lr, double beta1_comp,
                            double beta2_hat, double beta2_comp, double weight_decay, double eps, int decouple_lr,
                            double max_lr, int kahan_sum, int update_parameters, void* workspace, size_t workspace_bytes,
                            void* stream) {
  const bool update = update_parameters != 0;
  const bool kahan = update && kahan_sum && kahan_comps && low_precision(dtype);
  void* const* const lists[5] = {params, grads, exp_avgs, exp_avg_sqs, kahan ? kahan_comps : nullptr};
  const bool req[5] = {update, true, true, true, kahan};
  static const char* const names[5] = {"params", "grads", "exp_avgs", "exp_avg_sqs", "kahan_comps"};
  int rc = check_lists("optimi_b200_stableadamw", n, numels, dtype, 5, lists, req, names);
  if (rc != OPTIMI_OK || n == 0) return rc;
  if (update && weight_decay != 0 && decouple_lr && !(max_lr > 0))
    return fail(OPTIMI_ERR_INVALID_ARGUMENT, "optimi_b200_stableadamw: decouple_lr needs max_lr > 0");
  cudaStream_t s = (cudaStream_t)stream;
  switch (dtype) {
    case OPTIMI_F32:
      return stableadamw_typed<float>(n, params, grads, exp_avgs, exp_avg_sqs, kahan_comps, numels, lr, beta1_comp, beta2_hat,
                                      beta2_comp, weight_decay, eps, decouple_lr, max_lr, false, update, workspace,
                                      workspace_bytes, s);
    case OPTIMI_BF16:
      return stableadamw_typed<__nv_bfloat16>(n, params, grads, exp_avgs, exp_avg_sqs, kahan_comps, numels, lr, beta1_comp,
                                              beta2_hat, beta2_comp, weight_decay, eps, decouple_lr, max_lr, kahan, update,
                                              workspace, workspace_bytes, s);
    default:
      return stableadamw_typed<__half>(n, params, grads, exp_avgs, exp_avg_sqs, kahan_comps, numels, lr, beta1_comp, beta2_hat,
                                       beta2_comp, weight_decay, eps, decouple_lr, max_lr, kahan, update, workspace,
                                       workspace_bytes, s);
  }
}

size_t optimi_b200_grad_clip_workspace_bytes(int n, const int64_t* numels) {
  if (n <= 0 || !numels) return 16;
  constexpr int tile = tile_of<float, SumSqOp>();  // the float32 tile is the smallest
  return align_up((size_t)n * sizeof(float), 16) + (size_t)count_tiles(n, numels, tile) * sizeof(double) + 16;
}

void optimi_b200_grad_scale_begin(const float* device_factor) { g_grad_factor = device_factor; }

void optimi_b200_grad_scale_end(void) { g_grad_factor = nullptr; }

int optimi_b200_grad_clip_factor(int n, void* const* grads, const int64_t* numels, int dtype, double max_norm, float* out,
                                 void* workspace, size_t workspace_bytes, void* stream) {
  const char* fn = "optimi_b200_grad_clip_factor";
  void* const* const lists[2] = {grads, nullptr};
  const bool req[2] = {true, false};
  static const char* const names[2] = {"grads", ""};
  int rc = check_lists(fn, n, numels, dtype, 2, lists, req, names);
  if (rc != OPTIMI_OK) return rc;
  if (!out) return fail(OPTIMI_ERR_INVALID_ARGUMENT, "%s: out is NULL", fn);
  if (n == 0) return fail(OPTIMI_ERR_INVALID_ARGUMENT, "%s: no tensors", fn);
  const size_t need = optimi_b200_grad_clip_workspace_bytes(n, numels) - 16;
  if (!workspace || workspace_bytes < need)
    return fail(OPTIMI_ERR_WORKSPACE_TOO_SMALL, "%s: workspace of %zu bytes given, %zu needed", fn,
                workspace ? workspace_bytes : (size_t)0, need);
  if (reinterpret_cast<uintptr_t>(workspace) & 15) return fail(OPTIMI_ERR_INVALID_ARGUMENT, "%s: workspace is not 16-byte aligned", fn);
  float* tensor_norms = reinterpret_cast<float*>(workspace);
  double* partial = reinterpret_cast<double*>(reinterpret_cast<char*>(workspace) + align_up((size_t)n * sizeof(float), 16));
  cudaStream_t s = (cudaStream_t)stream;
  auto typed = [&](auto tag) {
    using T = decltype(tag);
    auto pass = [&](auto small) {
      constexpr bool SMALL = decltype(small)::value;
      return for_each_table<2, SMALL>(n, numels, lists, tile_of<T, SumSqOp>(), [&](const MtaTable<2, SMALL>& tab, int tiles) {
        int r = launch_kernel(fn, tile_sum_kernel<T, SumSqOp, SMALL>, tiles, kThreads, s, tab, SumSqArgs{}, partial);
        if (r != OPTIMI_OK) return r;
        const double* partial_in = partial;
        return launch_kernel(fn, norm_finalize_kernel<T, SMALL>, tab.n_tensors, 256, s, tab, partial_in, tensor_norms);
      });
    };
    // tensors without elements launch nothing: their norm is zero
    if (g_graph.mode != kGraphUpdate) {
      cudaError_t e = cudaMemsetAsync(tensor_norms, 0, (size_t)n * sizeof(float), s);
      if (e != cudaSuccess) return fail(OPTIMI_ERR_CUDA, "%s: cudaMemsetAsync: %s", fn, cudaGetErrorString(e));
    }
    int r = n <= MtaTable<2, true>::CAP ? pass(std::true_type{}) : pass(std::false_type{});
    if (r != OPTIMI_OK) return r;
    const float* norms_in = tensor_norms;
    return launch_kernel(fn, clip_factor_kernel<T>, 1, 256, s, norms_in, n, (float)max_norm, out);
  };
  switch (dtype) {
    case OPTIMI_F32: return typed(float{});
    case OPTIMI_BF16: return typed(__nv_bfloat16{});
    default: return typed(__half{});
  }
}

int optimi_b200_grad_sumsq(int n, void* const* grads, const int64_t* numels, int dtype, double* sumsq, void* workspace,
                           size_t workspace_bytes, void* stream) {
  const char* fn = "optimi_b200_grad_sumsq";
  void* const* const lists[2] = {grads, nullptr};
  const bool req[2] = {true, false};
  static const char* const names[2] = {"grads", ""};
  int rc = check_lists(fn, n, numels, dtype, 2, lists, req, names);
  if (rc != OPTIMI_OK || n == 0) return rc;
  if (!sumsq) return fail(OPTIMI_ERR_INVALID_ARGUMENT, "%s: sumsq is NULL", fn);
  const size_t need = optimi_b200_grad_clip_workspace_bytes(n, numels) - 16;
  if (!workspace || workspace_bytes < need)
    return fail(OPTIMI_ERR_WORKSPACE_TOO_SMALL, "%s: workspace of %zu bytes given, %zu needed", fn,
                workspace ? workspace_bytes : (size_t)0, need);
  if (reinterpret_cast<uintptr_t>(workspace) & 15) return fail(OPTIMI_ERR_INVALID_ARGUMENT, "%s: workspace is not 16-byte aligned", fn);
  double* partial = reinterpret_cast<double*>(workspace);
  cudaStream_t s = (cudaStream_t)stream;
  if (g_graph.mode != kGraphUpdate) {  // tensors without elements launch nothing: their sum is zero
    cudaError_t e = cudaMemsetAsync(sumsq, 0, (size_t)n * sizeof(double), s);
    if (e != cudaSuccess) return fail(OPTIMI_ERR_CUDA, "%s: cudaMemsetAsync: %s", fn, cudaGetErrorString(e));
  }
  auto typed = [&](auto tag) {
    using T = decltype(tag);
    auto pass = [&](auto small) {
      constexpr bool SMALL = decltype(small)::value;
      return for_each_table<2, SMALL>(n, numels, lists, tile_of<T, SumSqOp>(), [&](const MtaTable<2, SMALL>& tab, int tiles) {
        int r = launch_kernel(fn, tile_sum_kernel<T, SumSqOp, SMALL>, tiles, kThreads, s, tab, SumSqArgs{}, partial);
        if (r != OPTIMI_OK) return r;
        const double* partial_in = partial;
        return launch_kernel(fn, sumsq_finalize_kernel<SMALL>, tab.n_tensors, 256, s, tab, partial_in, sumsq);
      });
    };
    return n <= MtaTable<2, true>::CAP ? pass(std::true_type{}) : pass(std::false_type{});
  };
  switch (dtype) {
    case OPTIMI_F32: return typed(float{});
    case OPTIMI_BF16: return typed(__nv_bfloat16{});
    default: return typed(__half{});
  }
}

int optimi_b200_grad_norms_from_sumsq(int n, const double* sumsq, int dtype, float* norms, void* stream) {
  const char* fn = "optimi_b200_grad_norms_from_sumsq";
  if (n < 0) return fail(OPTIMI_ERR_INVALID_ARGUMENT, "%s: n_tensors=%d is negative", fn, n);
  if (n == 0) return OPTIMI_OK;
  if (!sumsq || !norms) return fail(OPTIMI_ERR_INVALID_ARGUMENT, "%s: sumsq or norms is NULL", fn);
  cudaStream_t s = (cudaStream_t)stream;
  const unsigned grid = (unsigned)((n + 255) / 256);
  switch (dtype) {
    case OPTIMI_F32: return launch_kernel(fn, norms_from_sumsq_kernel<float>, grid, 256, s, sumsq, n, norms);
    case OPTIMI_BF16: return launch_kernel(fn, norms_from_sumsq_kernel<__nv_bfloat16>, grid, 256, s, sumsq, n, norms);
    case OPTIMI_F16: return launch_kernel(fn, norms_from_sumsq_kernel<__half>, grid, 256, s, sumsq, n, norms);
  }
  return fail(OPTIMI_ERR_INVALID_ARGUMENT, "%s: unknown dtype code %d", fn, dtype);
}

int optimi_b200_clip_factor_from_norms(int n, const float* norms, int dtype, double max_norm, float* out, void* stream) {
  const char* fn = "optimi_b200_clip_factor_from_norms";
  if (n <= 0) return fail(OPTIMI_ERR_INVALID_ARGUMENT, "%s: no tensors", fn);
  if (!norms || !out) return fail(OPTIMI_ERR_INVALID_ARGUMENT, "%s: norms or out is NULL", fn);
  cudaStream_t s = (cudaStream_t)stream;
  switch (dtype) {
    case OPTIMI_F32: return launch_kernel(fn, clip_factor_kernel<float>, 1, 256, s, norms, n, (float)max_norm, out);
    case OPTIMI_BF16: return launch_kernel(fn, clip_factor_kernel<__nv_bfloat16>, 1, 256, s, norms, n, (float)max_norm, out);
    case OPTIMI_F16: return launch_kernel(fn, clip_factor_kernel<__half>, 1, 256, s, norms, n, (float)max_norm, out);
  }
  return fail(OPTIMI_ERR_INVALID_ARGUMENT, "%s: unknown dtype code %d", fn, dtype);
}

#endif  // part 2 (continues below with the static-scratch variant)

}  // extern "C"

#if OPTIMI_IN_PART(2)
// ---------------------------------------------------------------------------------------------
// StableAdamW without any caller-provided scratch
// ---------------------------------------------------------------------------------------------
namespace optimi {

// Scratch that lives in the library image itself.  The name below is only a host-side handle: the
// device address is looked up once per device with cudaGetSymbolAddress and that pointer is what
// the kernels receive.
static __device__ __align__(256) unsigned char g_static_scratch[OPTIMI_B200_STATIC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
static std::mutex g_static_scratch_mutex;
static void* g_static_scratch_ptr[kMaxDevices] = {};

static int static_scratch_of_current_device(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(OPTIMI_ERR_CUDA, "optimi_b200_stableadamw_static: cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices)
    return fail(OPTIMI_ERR_INVALID_ARGUMENT, "optimi_b200_stableadamw_static: device index %d is outside 0..%d", dev, kMaxDevices - 1);
  std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
  if (!g_static_scratch_ptr[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess || !p)
      return fail(OPTIMI_ERR_CUDA, "optimi_b200_stableadamw_static: cudaGetSymbolAddress on device %d: %s", dev, cudaGetErrorString(e));
    g_static_scratch_ptr[dev] = p;
  }
  *out = g_static_scratch_ptr[dev];
  return OPTIMI_OK;
}

template <typename T>
static size_t stable_scratch_need(int n, const int64_t* numels) {
  return align_up((size_t)n * sizeof(float2), 16) + (size_t)count_tiles(n, numels, tile_of<T, StableMomentsOp<true>>()) * sizeof(double);
}

}  // namespace optimi

extern "C" int optimi_b200_stableadamw_static(int n, void* const* params, void* const* grads, void* const* exp_avgs,
                                              void* const* exp_avg_sqs, void* const* kahan_comps, const int64_t* numels,
                                              int dtype, double lr, double beta1_comp, double beta2_hat, double beta2_comp,
                                              double weight_decay, double eps, int decouple_lr, double max_lr, int kahan_sum,
                                              int update_parameters, void* stream) {
  const char* fn = "optimi_b200_stableadamw_static";
  const bool update = update_parameters != 0;
  const bool kahan = update && kahan_sum && kahan_comps && low_precision(dtype);
  void* const* const lists[5] = {params, grads, exp_avgs, exp_avg_sqs, kahan ? kahan_comps : nullptr};
  const bool req[5] = {update, true, true, true, kahan};
  static const char* const names[5] = {"params", "grads", "exp_avgs", "exp_avg_sqs", "kahan_comps"};
  int rc = check_lists(fn, n, numels, dtype, 5, lists, req, names);
  if (rc != OPTIMI_OK || n == 0) return rc;
  if (update && weight_decay != 0 && decouple_lr && !(max_lr > 0))
    return fail(OPTIMI_ERR_INVALID_ARGUMENT, "%s: decouple_lr needs max_lr > 0", fn);

  void* scratch = nullptr;
  if (update) {  // the accumulate-only micro-step needs no scratch at all
    const size_t need = dtype == OPTIMI_F32    ? stable_scratch_need<float>(n, numels)
                        : dtype == OPTIMI_BF16 ? stable_scratch_need<__nv_bfloat16>(n, numels)
                                               : stable_scratch_need<__half>(n, numels);
    if (need > (size_t)OPTIMI_B200_STATIC_SCRATCH_BYTES)
      return fail(OPTIMI_ERR_WORKSPACE_TOO_SMALL,
                  "%s: this tensor list needs %zu bytes of scratch, the built-in scratch holds %zu; split the list into "
                  "several calls or use optimi_b200_stableadamw with your own workspace",
                  fn, need, (size_t)OPTIMI_B200_STATIC_SCRATCH_BYTES);
    rc = static_scratch_of_current_device(&scratch);
    if (rc != OPTIMI_OK) return rc;
  }
  cudaStream_t s = (cudaStream_t)stream;
  const size_t cap = (size_t)OPTIMI_B200_STATIC_SCRATCH_BYTES;
  switch (dtype) {
    case OPTIMI_F32:
      return stableadamw_typed<float>(n, params, grads, exp_avgs, exp_avg_sqs, kahan_comps, numels, lr, beta1_comp, beta2_hat,
                                      beta2_comp, weight_decay, eps, decouple_lr, max_lr, false, update, scratch, cap, s);
    case OPTIMI_BF16:
      return stableadamw_typed<__nv_bfloat16>(n, params, grads, exp_avgs, exp_avg_sqs, kahan_comps, numels, lr, beta1_comp,
                                              beta2_hat, beta2_comp, weight_decay, eps, decouple_lr, max_lr, kahan, update,
                                              scratch, cap, s);
    default:
      return stableadamw_typed<__half>(n, params, grads, exp_avgs, exp_avg_sqs, kahan_comps, numels, lr, beta1_comp, beta2_hat,
                                       beta2_comp, weight_decay, eps, decouple_lr, max_lr, kahan, update, scratch, cap, s);
  }
}
#endif  // part 2
