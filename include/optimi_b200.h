/* optimi_b200 — C ABI of the B200 (sm_100a) optimizer-step kernels.
 *
 * Each entry point replaces one of the reference's step back ends (the `_foreach_*`,
 * `_single_param_*` and `_triton_*` functions its functional API dispatches to) for a whole list
 * of tensors in one or a few kernel launches.  Conventions shared by every entry point:
 *
 *   - `n_tensors` tensors; `numels[i]` is the element count of tensor i (host array).
 *   - Every `void* const* xs` is a HOST array of `n_tensors` DEVICE pointers.  All tensors of one
 *     call live on the current device, are contiguous, and share one storage type `dtype`
 *     (OPTIMI_F32 / OPTIMI_BF16 / OPTIMI_F16).  Parameters, gradients and states of a tensor
 *     have the same element count.
 *   - Everything is updated in place.  Gradients are only read (the reference's foreach path
 *     leaves them clobbered; callers of either must not reuse them after the step).
 *   - Scalars arrive as the doubles the reference's functional layer computes on the host
 *     (debiased betas, folded weight-decay factor, ...) and are narrowed to fp32 inside, exactly
 *     where the reference's ATen ops narrow them.
 *   - Arithmetic replays the reference's op sequence in registers: one fp32 computation and one
 *     rounding to the storage type per ATen op, so low-precision results are bit-identical to
 *     the reference's foreach path on the same device (StableAdamW up to the summation order of
 *     its per-tensor mean).
 *   - `kahan_comps == NULL` (or kahan_sum == 0) selects the plain update.
 *   - `update_parameters == 0` is the optimizer-accumulation micro-step: state averages advance,
 *     weight decay and the parameter update are skipped, parameters and Kahan buffers untouched.
 *   - `stream` is a cudaStream_t (NULL = the legacy default stream).  Calls only enqueue work.
 *   - Return value: OPTIMI_OK or a negative OPTIMI_ERR_*; optimi_b200_last_error() gives the text
 *     of the calling thread's last failure.  Nothing aborts, nothing traps on the device.
 *   - No entry point allocates or frees device memory.
 */
#ifndef OPTIMI_B200_H
#define OPTIMI_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define OPTIMI_F32 0
#define OPTIMI_BF16 1
#define OPTIMI_F16 2

#define OPTIMI_OK 0
#define OPTIMI_ERR_INVALID_ARGUMENT (-1)
#define OPTIMI_ERR_CUDA (-2)
#define OPTIMI_ERR_WORKSPACE_TOO_SMALL (-3)
#define OPTIMI_ERR_CAPTURE (-4) /* a launch met a capturing stream outside a record bracket, or the reverse */

const char* optimi_b200_last_error(void);

/* Library version as major*10000 + minor*100 + patch. */
int optimi_b200_version(void);

/* Number of CUDA kernels this library has launched in the calling process so far (all threads). */
unsigned long long optimi_b200_launch_count(void);

/* Steps inside a CUDA graph.  No counterpart in the reference (its kernels are launched eagerly
 * from Python every step).
 *
 * Every kernel of this library takes its scalars by value, and most of them change from step to
 * step (bias corrections, a scheduled learning rate, Ranger's lookahead flag), so a step that was
 * merely captured would replay stale scalars.  A step entry point therefore refuses a capturing
 * stream (OPTIMI_ERR_CAPTURE) unless the calling thread has opened a record bracket:
 *
 *   capture time   optimi_b200_graph_record_begin();
 *                  ... the step calls, on the capturing stream: launches are captured as usual and
 *                      the graph node of each is remembered ...
 *                  optimi_b200_graph_record_end(&nodes);
 *   every replay   optimi_b200_graph_update_begin(nodes, graph_exec);
 *                  ... THE SAME step calls in the same order with the coming step's scalars (and
 *                      pointers, which may differ): nothing is launched, each would-be launch
 *                      rewrites the kernel parameters of its node in `graph_exec`
 *                      (cudaGraphExecKernelNodeSetParams) ...
 *                  optimi_b200_graph_update_end();      then launch the graph
 *
 * `graph_exec` is the cudaGraphExec_t instantiated from the captured graph; the captured
 * cudaGraph_t must still exist while updates are made (its nodes name the ones to rewrite).  An
 * update only affects launches of the graph made after it.  The brackets are per thread and do
 * not nest; they have not been exercised together with the peer push / pull brackets below.  `nodes` is freed
 * with optimi_b200_graph_nodes_free (NULL is fine).  update_end fails if the step issued a
 * different number of launches than were recorded (the tensor list changed: capture again). */
typedef struct optimi_b200_graph_nodes optimi_b200_graph_nodes;
int optimi_b200_graph_record_begin(void);
int optimi_b200_graph_record_end(optimi_b200_graph_nodes** out);
int optimi_b200_graph_nodes_count(const optimi_b200_graph_nodes* nodes);
void optimi_b200_graph_nodes_free(optimi_b200_graph_nodes* nodes);
int optimi_b200_graph_update_begin(optimi_b200_graph_nodes* nodes, void* graph_exec);
int optimi_b200_graph_update_end(void);

/* Gradient scaling fused into the step.  No counterpart in the reference: its users clip the gradient
 * norm (torch.nn.utils.clip_grad_norm_) or unscale a loss scale (GradScaler.unscale_) in passes of
 * their own between backward and step(), each a full read and write of the gradients.
 *
 * optimi_b200_grad_scale_begin(factor): until _end, every launch the calling thread makes through
 * a step entry point multiplies each gradient element by the fp32 value at the DEVICE address
 * `factor` as it is loaded, g <- round_to_storage(g * factor) — the arithmetic of
 * torch._foreach_mul_(grads, factor_tensor) — and steps with that.  The gradient buffers are not
 * written.  The value is read when the kernels run, so it may be produced on the same stream just
 * before (optimi_b200_grad_clip_factor below, or a GradScaler's inverse scale).  Not combinable
 * with the gradient pull bracket (the peer push composes with it).
 *
 * optimi_b200_grad_clip_factor: writes out[0] = min(1, max_norm * (1 / (total + 1e-6))) and
 * out[1] = total, the 2-norm of all gradients, to the DEVICE array `out` (2 floats), following
 * clip_grad_norm_'s own order of operations and roundings (per-tensor norms in the storage type,
 * their 2-norm, reciprocal, product, clamp).  One read of the gradients; sums are taken in double
 * in a fixed order, so the result is deterministic and agrees with PyTorch's up to the rounding error of
 * its fp32 sums (bf16 / fp16: at most one unit of the storage type; fp32: a relative 1e-6 or so).
 * `workspace`: DEVICE scratch of
 * optimi_b200_grad_clip_workspace_bytes(n_tensors, numels) bytes, 16-byte aligned. */
void optimi_b200_grad_scale_begin(const float* device_factor);
void optimi_b200_grad_scale_end(void);
size_t optimi_b200_grad_clip_workspace_bytes(int n_tensors, const int64_t* numels);
int optimi_b200_grad_clip_factor(int n_tensors, void* const* grads, const int64_t* numels, int dtype, double max_norm,
                                 float* out, void* workspace, size_t workspace_bytes, void* stream);

/* The same clip factor in separable steps, for gradients that one call cannot see whole: tensors cut
 * into pieces that live on several ranks (ZeRO-1 sharding), or lists of several dtypes (float32
 * embeddings beside a bfloat16 body, as optimi's to_low_precision leaves a model:
 * optimi/utils.py:104-169).  No counterpart in the reference.
 *
 * optimi_b200_grad_sumsq: sumsq[i] (DEVICE, n_tensors doubles) = sum of squares of tensor (or piece) i,
 * in double, in a fixed order.  `workspace` as for optimi_b200_grad_clip_factor.  The caller adds up the
 * pieces of one tensor (and the ranks' contributions) as it sees fit.
 * optimi_b200_grad_norms_from_sumsq: norms[i] (DEVICE floats) = sqrt((float)sumsq[i]) rounded to the
 * storage type `dtype`, what torch._foreach_norm returns for a tensor of that dtype.
 * optimi_b200_clip_factor_from_norms: out[0] = min(1, max_norm * (1 / (total + 1e-6))), out[1] = total
 * = the 2-norm of `norms`, every intermediate rounded to `dtype` — the dtype torch promotes the stacked
 * norms to: the gradients' own if they share one, float32 otherwise. */
int optimi_b200_grad_sumsq(int n_tensors, void* const* grads, const int64_t* numels, int dtype, double* sumsq,
                           void* workspace, size_t workspace_bytes, void* stream);
int optimi_b200_grad_norms_from_sumsq(int n_tensors, const double* sumsq, int dtype, float* norms, void* stream);
int optimi_b200_clip_factor_from_norms(int n_tensors, const float* norms, int dtype, double max_norm, float* out,
                                       void* stream);

/* Adam / AdamW.  Replaces _foreach_adam (optimi/adam.py:399-453), _single_param_adam
 * (optimi/adam.py:354-396) and the Triton launchers (optimi/adam.py:533-630); called where
 * adam() picks its back end (optimi/adam.py:278-309).  `weight_decay` is the factor adam()
 * has already folded (1 - lr*wd or 1 - lr/max_lr*wd when decouple_wd != 0, the raw L2
 * coefficient otherwise; optimi/adam.py:269-273). */
int optimi_b200_adam(int n_tensors, void* const* params, void* const* grads, void* const* exp_avgs,
                     void* const* exp_avg_sqs, void* const* kahan_comps, const int64_t* numels, int dtype,
                     double lr, double beta1_comp, double beta2_hat, double beta2_comp, double weight_decay,
                     double eps, int decouple_wd, int kahan_sum, int update_parameters, void* stream);

/* Fusing the step with the parameter exchange of a sharded (ZeRO-1) run.  No counterpart in the
 * reference, which has no distributed code: it stands for "step this rank's shard, then all-gather
 * the updated parameters".  Every rank keeps the whole parameter buffer; `peer_deltas[j]`
 * (j < n_peers <= 7) is the byte distance from this rank's copy of that buffer to peer j's copy as
 * mapped into this process (e.g. the buffer pointers of a symmetric-memory allocation), a multiple
 * of 16.  Between optimi_b200_push_begin and optimi_b200_push_end every parameter-updating launch
 * the CALLING THREAD makes through any entry point of this library stores each updated parameter
 * vector locally and, with plain peer stores over NVLink, at the same offset in every peer's copy,
 * tile by tile as the step proceeds.  The kernels wait for nobody, so the caller orders the ranks on
 * BOTH sides of the launches (any stream-ordered collective or barrier will do): before them, so that
 * no peer is still reading the parameter buffer this rank is about to store into (its forward,
 * backward or evaluation pass must have finished on every rank), and after them, before the pushed
 * values are read on the peers.  Blocks start their round over the peers at different peers, so the
 * order of the entries of `peer_deltas` does not matter.  Accumulation-only steps
 * (update_parameters == 0) push nothing.  Composes with optimi_b200_grad_scale_begin (the gradients
 * are scaled on load, the parameters pushed on store). */
int optimi_b200_push_begin(int n_peers, const int64_t* peer_deltas);
void optimi_b200_push_end(void);

/* Fusing the gradient reduce-scatter of a data-parallel run into the step.  No counterpart in the
 * reference.  Every rank keeps its own full gradient buffer in memory the other ranks can read;
 * `grad_deltas[r]` (r < n_ranks <= 8, in rank order, 0 for the calling rank itself) is the byte
 * distance from this rank's gradient buffer to rank r's as mapped into this process, a multiple of
 * 16.  Between optimi_b200_pull_begin and optimi_b200_pull_end every launch the calling thread
 * makes reads, for each element it steps, the gradient of all n_ranks ranks, adds them in fp32 in
 * rank order, multiplies by `scale` (1/n_ranks for a mean) and rounds once to the storage type;
 * that value is the gradient the optimizer sees.  It exists only in registers; no rank's buffer is
 * written.  The kernels wait for nobody: the caller orders the ranks before the launch (all
 * gradients complete) and after it (before any gradient buffer is overwritten).  Combine with
 * optimi_b200_push_begin for reduce-scatter + step + all-gather in one kernel.  Not available for
 * StableAdamW (its launches are rejected while a pull is active). */
int optimi_b200_pull_begin(int n_ranks, const int64_t* grad_deltas, double scale);
void optimi_b200_pull_end(void);

/* Lion.  Replaces _foreach_lion (optimi/lion.py:341-380), _single_param_lion (optimi/lion.py:301-338)
 * and the Triton launchers (optimi/lion.py:453-530).  `weight_decay` is the folded factor
 * (optimi/lion.py:227-231), 0 for none. */
int optimi_b200_lion(int n_tensors, void* const* params, void* const* grads, void* const* exp_avgs,
                     void* const* kahan_comps, const int64_t* numels, int dtype, double lr, double beta1_comp,
                     double beta2_comp, double weight_decay, int kahan_sum, int update_parameters, void* stream);

/* SGD with optional momentum / dampening.  Replaces _foreach_sgd (optimi/sgd.py:375-421),
 * _single_param_sgd (optimi/sgd.py:329-372) and the Triton launchers (optimi/sgd.py:501-584).
 * `exp_avgs` may be NULL when momentum == 0. */
int optimi_b200_sgd(int n_tensors, void* const* params, void* const* grads, void* const* exp_avgs,
                    void* const* kahan_comps, const int64_t* numels, int dtype, double lr, double momentum,
                    double weight_decay, int dampening, int decouple_wd, int kahan_sum, int update_parameters,
                    void* stream);

/* StableAdamW.  Replaces _foreach_stableadamw (optimi/stableadamw.py:475-544),
 * _single_param_stableadamw (optimi/stableadamw.py:421-472) and the two Triton kernels with
 * their launchers (optimi/stableadamw.py:551-791).  The per-tensor RMS never leaves the device:
 * pass A advances the averages and writes one partial sum per tile, a one-block-per-tensor
 * pass folds them in a fixed order into the clipped learning rate and weight-decay factor, pass
 * B applies the update.  `weight_decay` is the RAW coefficient and `max_lr` the scheduled
 * maximum (used when decouple_lr != 0), because the factor depends on the clipped learning
 * rate (optimi/stableadamw.py:512-524).  `workspace` is device scratch of at least
 * optimi_b200_stableadamw_workspace_bytes(...) bytes, 16-byte aligned; its contents need not be
 * initialised and are overwritten. */
size_t optimi_b200_stableadamw_workspace_bytes(int n_tensors, const int64_t* numels);
int optimi_b200_stableadamw(int n_tensors, void* const* params, void* const* grads, void* const* exp_avgs,
                            void* const* exp_avg_sqs, void* const* kahan_comps, const int64_t* numels, int dtype,
                            double lr, double beta1_comp, double beta2_hat, double beta2_comp, double weight_decay,
                            double eps, int decouple_lr, double max_lr, int kahan_sum, int update_parameters,
                            void* workspace, size_t workspace_bytes, void* stream);

/* StableAdamW for callers that have no device memory to hand over.  No counterpart in the reference:
 * its StableAdamW keeps its scratch in ordinary PyTorch tensors and never faces the question.
 *
 * Who this is for: code that gets the parameter, gradient and state pointers from somebody else and
 * has no allocator of its own to call — a plugin inside a runtime that owns all device memory and
 * forbids cudaMalloc after start-up, a step running where an allocation is not allowed to happen
 * (cudaMalloc synchronises the whole device and can fail under memory pressure, which a training
 * loop that has planned its memory to the last gigabyte cannot tolerate), or a binding in a
 * language whose CUDA wrapper exposes launches but not allocation.  Such a caller cannot satisfy
 * the `workspace` argument of optimi_b200_stableadamw.  Here the scratch is a fixed array of
 * OPTIMI_B200_STATIC_SCRATCH_BYTES inside the library image; every GPU that loads the library
 * carries it until the process exits.
 *
 * Same arguments and results as optimi_b200_stableadamw without `workspace`/`workspace_bytes`
 * (results are bit-identical for the same inputs).  Limits and rules:
 *   - The list must need no more scratch than the array holds: 8 bytes per tensor plus 8 bytes per
 *     tile of 1024 (bf16/fp16) or 512 (fp32) elements, i.e. about 536 M bf16 or 268 M fp32 elements
 *     per call.  Larger lists are rejected with OPTIMI_ERR_WORKSPACE_TOO_SMALL before anything is
 *     launched; split them into several calls (the optimizer is per-tensor, so that is exact).
 *   - The first call on each device looks up the array's device address (cudaGetSymbolAddress, with
 *     that device current).  Make that first call outside any stream capture.
 *   - All calls on a device share the one array and it keeps the previous call's contents.  Nothing
 *     in it has to start at zero (every slot is written before it is read within a call), but two
 *     calls that overlap on the GPU — different streams without an ordering between them — race
 *     on it.  Calls on one stream, or ordered by events, are fine.
 *   - Calls cudaMalloc, cudaFree or any allocating routine: never. */
#define OPTIMI_B200_STATIC_SCRATCH_BYTES (4u << 20)
int optimi_b200_stableadamw_static(int n_tensors, void* const* params, void* const* grads, void* const* exp_avgs,
                                   void* const* exp_avg_sqs, void* const* kahan_comps, const int64_t* numels, int dtype,
                                   double lr, double beta1_comp, double beta2_hat, double beta2_comp, double weight_decay,
                                   double eps, int decouple_lr, double max_lr, int kahan_sum, int update_parameters,
                                   void* stream);

/* Adan.  Replaces _foreach_adan (optimi/adan.py:472-546), _single_param_adan (optimi/adan.py:405-469)
 * and the Triton launchers (optimi/adan.py:652-770).  `prev_grads` holds the NEGATED previous
 * gradient (optimi/adan.py:109).  `weight_decay` is the folded factor 1 + lr*wd (Adan style,
 * applied by division) or 1 - lr*wd (adam_wd != 0, applied by multiplication), 0 for none
 * (optimi/adan.py:300-309). */
int optimi_b200_adan(int n_tensors, void* const* params, void* const* grads, void* const* exp_avgs,
                     void* const* exp_avg_diffs, void* const* exp_avg_sqs, void* const* prev_grads,
                     void* const* kahan_comps, const int64_t* numels, int dtype, double lr, double beta1_comp,
                     double beta2, double beta2_comp, double beta3_hat, double beta3_comp, double eps,
                     double weight_decay, int adam_wd, int kahan_sum, int update_parameters, void* stream);

/* RAdam.  Replaces _foreach_radam (optimi/radam.py:420-479), _single_param_radam
 * (optimi/radam.py:368-417) and the Triton launchers (optimi/radam.py:567-686).
 * `use_rect == 0` is the reference's rect=None (rho <= 5): momentum-only step. */
int optimi_b200_radam(int n_tensors, void* const* params, void* const* grads, void* const* exp_avgs,
                      void* const* exp_avg_sqs, void* const* kahan_comps, const int64_t* numels, int dtype,
                      double lr, double beta1_comp, double beta2_hat, double beta2_comp, double weight_decay,
                      double eps, int use_rect, double rect, int decouple_wd, int kahan_sum, int update_parameters,
                      void* stream);

/* Ranger (RAdam + Lookahead).  Replaces _foreach_ranger (optimi/ranger.py:476-561),
 * _single_param_ranger (optimi/ranger.py:402-473) and the Triton launchers
 * (optimi/ranger.py:674-810).  `do_lookahead != 0` on every k-th step (step % k == 0,
 * optimi/ranger.py:537); the Kahan lookahead follows the foreach and Triton variants, which do
 * not scale the slow-weight error by alpha. */
int optimi_b200_ranger(int n_tensors, void* const* params, void* const* grads, void* const* exp_avgs,
                       void* const* exp_avg_sqs, void* const* la_params, void* const* kahan_comps,
                       const int64_t* numels, int dtype, double lr, double beta1_comp, double beta2_hat,
                       double beta2_comp, double weight_decay, double eps, int use_rect, double rect,
                       int do_lookahead, double alpha, int decouple_wd, int kahan_sum, int update_parameters,
                       void* stream);

#ifdef __cplusplus
}
#endif
#endif /* OPTIMI_B200_H */
