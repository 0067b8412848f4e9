/*
 * ps_b200.h — C ABI of the B200 (sm_100a) chunk optimizer step.
 *
 * The library replaces the native half of PatrickStar's mixed-precision
 * optimizer step: the pybind module `cpu_adam_op` (create_adam / adam_update /
 * destroy_adam, patrickstar/ops/csrc/adam/cpu_adam.cpp:751-756) and the
 * per-chunk work that patrickstar/ops/fp16_cpu_adam.py and
 * patrickstar/ops/chunk_io_buff.py wrap around it (fp16 grad chunk read,
 * fp32 -> fp16 param chunk write-back, overflow gate, loss-scale update).
 *
 * Conventions
 *   - plain C: pointers, sizes, scalars.  No torch, no C++ types.
 *   - every pointer named *_dev is a device address (cudaMalloc'ed or pinned
 *     host memory mapped into the device address space); the library never
 *     allocates or frees device memory behind these calls.
 *   - `stream` is a cudaStream_t passed as void*; NULL is the legacy default
 *     stream.  All device work is enqueued on it and nothing synchronises
 *     unless the comment of a function says so.
 *   - return value: 0 on success, a negative PS_ERR_* code otherwise.  Nothing
 *     throws, traps or aborts.  (The reference always returns 0, ignores CUDA
 *     return codes and dereferences a null pointer on an unknown optimizer id,
 *     cpu_adam.cpp:721-722; here those cases are reported.)
 *   - there is no CPU fallback: without a CUDA device every compute entry
 *     point returns PS_ERR_CUDA.
 */
#ifndef PS_B200_H
#define PS_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PS_OK 0
#define PS_ERR_INVALID (-1)    /* null pointer, bad size, bad hyper-parameter */
#define PS_ERR_UNKNOWN_ID (-2) /* optimizer id was never created / already destroyed */
#define PS_ERR_ALIGN (-3)      /* a pointer or offset breaks the stated alignment rule */
#define PS_ERR_CUDA (-4)       /* a CUDA runtime call failed; see ps_last_cuda_error() */
#define PS_ERR_TABLE (-5)      /* chunk / segment table failed validation */
#define PS_ERR_LIMIT (-6)      /* a stated maximum (groups, slots, static capacity) exceeded */

#define PS_MAX_GROUPS 15              /* hyper-parameter groups per optimizer */
#define PS_MAX_SLOTS (PS_MAX_GROUPS + 1) /* slot 0 = first call of a step, 1+g = later calls of group g */

/* One local chunk.  Mirrors what the reference keeps per chunk id: the fp16
 * param chunk whose storage the gradients reuse (patrickstar/core/hook.py:214-216)
 * and the fp32 master / momentum / variance chunks laid out like it
 * (patrickstar/ops/fp16_cpu_adam.py:132-170).  All four base pointers must be
 * 16-byte aligned.  Elements outside every segment are left untouched. */
typedef struct ps_chunk_desc {
    float* p32;        /* fp32 master params, updated in place                  */
    float* exp_avg;    /* fp32 momentum, updated in place                       */
    float* exp_avg_sq; /* fp32 variance, updated in place                       */
    uint16_t* h16;     /* fp16 slot: gradients on entry, updated params on exit */
    uint32_t numel;    /* elements in use (<= chunk capacity)                   */
    uint32_t seg_begin; /* [seg_begin, seg_end) in the segment table            */
    uint32_t seg_end;
    uint32_t reserved; /* ps_chunk_step only: first element to process (a multiple of 2048;
                          0 = whole chunk).  Lets a launch cover the piece [first, numel) of a
                          chunk whose p32 / exp_avg / exp_avg_sq pointers are biased so that
                          index `first` is the first staged element (offload pipeline).       */
} ps_chunk_desc;

/* A run of elements of one chunk that shares hyper-parameters: [start, end)
 * in chunk-local element offsets, sorted and non-overlapping within a chunk.
 * `slot` selects the ps_hyper_slot the step-begin kernel prepared. */
typedef struct ps_segment {
    uint32_t start;
    uint32_t end;
    uint32_t slot;
    uint32_t reserved;
} ps_segment;

/* Hyper-parameters of one param group, as FP16Adam keeps them per parameter
 * (patrickstar/ops/fp16_cpu_adam.py:112-120). */
typedef struct ps_group_hyper {
    float lr, beta1, beta2, eps, weight_decay;
    int32_t adamw_mode;
    int32_t reserved[2];
} ps_group_hyper;

/* What one step needs besides the tables.  `first_group` is the group of the
 * first segment the rank visits in a step and `last_group` that of the last
 * one; `n_calls` is the number of segments (the reference makes one
 * adam_update call per tensor, and its beta^t depends on that call history,
 * patrickstar/ops/csrc/includes/cpu_adam.h:143-162). */
typedef struct ps_step_plan {
    double clip;         /* gradient_clipping of FP16Adam; <= 0 disables (fp16_cpu_adam.py:365-379) */
    ps_group_hyper groups[PS_MAX_GROUPS];
    int32_t n_groups;
    int32_t first_group;
    int32_t last_group;
    int32_t n_calls;
    float grad_divisor;  /* world size when the fp16 `payload /= world_size` of
                            patrickstar/core/client.py:838 is folded into the load; <= 1 disables */
    int32_t bias_correction;
} ps_step_plan;

/* Device-resident loss-scaler state: the fields of DynamicLossScaler
 * (patrickstar/fp16/loss_scaler.py:107-124) with Python's float as double and
 * Python's int as int64.  dynamic == 0 is the static LossScaler (:46-76),
 * dynamic < 0 means "no loss scaler" (loss_scale -1 in ds_cpu_adam_update). */
typedef struct ps_scaler_state {
    double cur_scale;
    double scale_factor;
    double min_scale;
    int64_t cur_iter;
    int64_t last_overflow_iter;
    int64_t scale_window;
    int32_t delayed_shift;
    int32_t cur_hysteresis;
    int32_t consecutive_hysteresis;
    int32_t dynamic;
} ps_scaler_state;

/* Derived per-slot constants, prepared on the device by ps_step_begin exactly
 * as Adam_Optimizer::Step derives them (cpu_adam.cpp:42-46). */
typedef struct ps_hyper_slot {
    float loss_scale; /* <= 0: no unscale */
    float beta1, beta2, beta1_minus1, beta2_minus1;
    float bias2_sqrt, eps, step_size;
    float weight_decay, w_decay;
    float clip;         /* already min(65504, clip * scale); <= 0 disabled */
    float grad_divisor; /* <= 1 disabled */
    int32_t adamw_mode;
    float inv_loss_scale; /* 1 / loss_scale when the scale is a power of two (the product is then
                             bit-identical to the division), else 0 = divide */
    float inv_grad_divisor; /* float(1 / grad_divisor): torch computes the fp16 `payload /= world_size`
                               on a CUDA tensor as half(float(g) * (1.0f / world)); 0 = derive it in the
                               kernel */
    int32_t reserved;
} ps_hyper_slot;

/* Device-resident control block of one optimizer (one per FP16Adam object). */
typedef struct ps_step_ctrl {
    int32_t skip;          /* set by ps_step_begin: 1 = this step is skipped */
    int32_t error;         /* sticky device-side error word (0 = none)       */
    uint64_t step;         /* state["step"]: counts non-skipped steps        */
    uint64_t n_skipped;    /* total skipped steps                            */
    /* emulation of Adam_Optimizer's call-history state (cpu_adam.h:143-162) */
    uint64_t native_step;
    float betta1, betta2, betta1_t, betta2_t;
    ps_hyper_slot slots[PS_MAX_SLOTS];
} ps_step_ctrl;

/* ------------------------------------------------------------------ */
/* library                                                              */
/* ------------------------------------------------------------------ */
int ps_version(void);
const char* ps_strerror(int code);
int ps_last_cuda_error(void); /* cudaError_t of the last failed runtime call on this thread */

/* ------------------------------------------------------------------ */
/* tensor-level API: 1:1 image of the cpu_adam_op module                */
/* ------------------------------------------------------------------ */

/* create_adam (cpu_adam.cpp:379-417).  Host-only. */
int ps_adam_create(int optimizer_id, float alpha, float betta1, float betta2, float eps,
                   float weight_decay, int adamw_mode, int should_log);

/* destroy_adam (cpu_adam.cpp:744-749).  Host-only. */
int ps_adam_destroy(int optimizer_id);

/* adam_update / ds_adam_step (cpu_adam.cpp:700-742) on device pointers.
 * params/exp_avg/exp_avg_sq: fp32 [n], updated in place.  grads: fp16 bits
 * (g_is_half != 0) or fp32, read-only.  loss_scale <= 0: no unscale.
 * p16_out (may be NULL): receives half(params) — the write-back the reference
 * does as a separate chunk copy (patrickstar/ops/chunk_io_buff.py:85-128); it
 * may alias `grads`.  Pointers need only their natural alignment; when the
 * four of them are not mutually 16-byte co-aligned a slower element-wise
 * kernel is used. */
int ps_adam_update(int optimizer_id, size_t step, float lr, float beta1, float beta2, float epsilon,
                   float weight_decay, int bias_correction, float* params_dev, const void* grads_dev,
                   float* exp_avg_dev, float* exp_avg_sq_dev, size_t n, int g_is_half,
                   float loss_scale, uint16_t* p16_out_dev, void* stream);

/* Host-only: beta1^t, beta2^t, bias_correction1, bias_correction2 and the step
 * the optimizer object holds after its last ps_adam_update (for tests). */
int ps_adam_get_state(int optimizer_id, float out[4], uint64_t* step);

/* ------------------------------------------------------------------ */
/* chunk-level API: what FP16Adam.step drives                           */
/* ------------------------------------------------------------------ */

/* Host-side validation of a chunk table and its segment table before they are
 * uploaded: 16-byte aligned non-null bases, numel <= chunk_capacity, `reserved`
 * (first element) a multiple of 2048 and below numel (0 for an empty chunk),
 * segments sorted, non-overlapping, inside numel, slot < n_slots. */
int ps_table_check(const ps_chunk_desc* chunks_host, uint32_t n_chunks, const ps_segment* segs_host,
                   uint32_t n_segs, uint32_t n_slots, uint32_t chunk_capacity);

/* Host-side validation of descriptors that cover a PIECE [reserved, numel) of a
 * chunk (the offload pipeline's rows, see ps_offload_chunk): non-null 16-byte
 * aligned bases, reserved a multiple of 2048 and below numel <= chunk_capacity,
 * a non-empty segment range inside the table.  The segments are the whole
 * chunk's (already validated with ps_table_check) and may reach beyond the
 * piece; the kernel clips them to [reserved, numel). */
int ps_piece_table_check(const ps_chunk_desc* pieces_host, uint32_t n_pieces, uint32_t n_segs,
                         uint32_t chunk_capacity);

/* Host-only helper: out[2*i] = float(pow(double(beta1), t0+i)), out[2*i+1] the
 * same for beta2 — the values IncrementStep's pow branch produces
 * (cpu_adam.h:147-156).  The step-begin kernel looks them up by the
 * device-resident step counter. */
int ps_pow_table_fill(float beta1, float beta2, uint64_t t0, uint64_t count, float* out_host);

/* Initialise a control block on the device (step counter, beta history).
 * Enqueues one small kernel. */
int ps_ctrl_init(ps_step_ctrl* ctrl_dev, uint64_t step, float betta1, float betta2, void* stream);

/* Initialise a scaler state on the device from a host copy. */
int ps_scaler_init(ps_scaler_state* scaler_dev, const ps_scaler_state* init_host, void* stream);

/* Overflow scan — DynamicLossScaler._has_inf_or_nan (loss_scaler.py:133-155)
 * over the fp16 slot of every chunk of the table; ORs 1 into *flag_dev when an
 * inf or nan is found.  Read-only, 2 B/element. */
int ps_overflow_scan(const ps_chunk_desc* chunks_dev, uint32_t n_chunks, uint32_t max_numel,
                     int32_t* flag_dev, void* stream);

/* Same test on one plain fp16 buffer (FP16Adam.check_overflow on one grad). */
int ps_overflow_scan_buffer(const uint16_t* g_dev, size_t n, int32_t* flag_dev, void* stream);

/* Gradient hand-off of the backward pass — what the reference's post-backward
 * hook does per parameter with a host sync (patrickstar/core/hook.py:212-216:
 * check_overflow(param), then the gradient is copied into the parameter's fp16
 * slot in the chunk): one pass that copies grad_dev[0..n) into slot_dev[0..n)
 * and ORs 1 into *flag_dev (may be NULL: copy only) when an inf or nan is seen.
 * No synchronisation.  A step fed this way can skip its own overflow scan. */
int ps_grad_handoff(const uint16_t* grad_dev, uint16_t* slot_dev, size_t n, int32_t* flag_dev, void* stream);

/* Head of FP16Adam.step (fp16_cpu_adam.py:549-606, 624-625) as one
 * single-thread kernel, no host sync: reads *flag_dev (already MAX-reduced
 * over ranks); on overflow sets ctrl->skip, otherwise increments the step
 * counter, replays IncrementStep/update_state for the plan's calls using
 * pow_table_dev (pairs as written by ps_pow_table_fill for each group g at
 * pow_table_dev + 2*(g*pow_table_len + t)) and fills the hyper slots with the
 * scale in force for this step.  Then applies DynamicLossScaler.update_scale
 * (loss_scaler.py:158-182) and clears the flag. */
int ps_step_begin(ps_step_ctrl* ctrl_dev, ps_scaler_state* scaler_dev, int32_t* flag_dev,
                  const ps_step_plan* plan_host, const float* pow_table_dev, uint64_t pow_table_len,
                  void* stream);

/* DynamicLossScaler.update_scale (loss_scaler.py:158-182) alone, for callers that
 * drive the scaler themselves: overflow is *flag_dev != 0 when flag_dev is not
 * NULL (the flag is cleared afterwards), else `overflow_host`. */
int ps_scaler_update(ps_scaler_state* scaler_dev, int32_t* flag_dev, int overflow_host, void* stream);

/* The fused chunk step over a table of chunks, one launch.  When ctrl->skip is
 * 0: per element unscale the fp16 grad, Adam/AdamW on fp32 master, m, v in the
 * reference's operation order (cpu_adam.cpp:33-144), write half(master) into
 * the fp16 slot (28 B/element).  When ctrl->skip is 1: restore the fp16 slot
 * from the fp32 master (fp16_cpu_adam.py:298-309; 6 B/element). */
int ps_chunk_step(const ps_chunk_desc* chunks_dev, uint32_t n_chunks, uint32_t max_numel,
                  const ps_segment* segs_dev, const ps_step_ctrl* ctrl_dev, void* stream);

/* FP16Adam.has_overflow_and_reset_param's restore alone
 * (patrickstar/ops/fp16_cpu_adam.py:298-309): the fp16 slot of every segment of
 * every chunk of the table := half(fp32 master), 6 B/element, without a control
 * block.  (ps_chunk_step does the same when ctrl->skip is set.) */
int ps_restore_fp16(const ps_chunk_desc* chunks_dev, uint32_t n_chunks, uint32_t max_numel,
                    const ps_segment* segs_dev, void* stream);

/* One parameter that is managed by torch instead of the chunk list — the
 * reference's TORCH_BASED kind (the CPU-embedding weights,
 * patrickstar/core/preprocess.py:351-369): the parameter itself is the fp32
 * master, its gradient is fp32, there is no fp16 slot and no write-back
 * (patrickstar/ops/fp16_cpu_adam.py:345-353).  All pointers need 4-byte
 * alignment only; 16-byte aligned ones take a vector path. */
typedef struct ps_tensor_desc {
    float* p32;        /* the parameter, fp32, updated in place */
    const float* grad; /* its fp32 gradient, read-only          */
    float* exp_avg;
    float* exp_avg_sq;
    uint64_t numel;
    uint32_t slot;     /* ps_hyper_slot of its call in the step's call sequence */
    uint32_t reserved;
} ps_tensor_desc;

#define PS_TENSOR_TABLE_MAX 1024u /* rows per ps_tensor_table_step call */

/* The step for a table of such parameters, one launch, driven by the same
 * control block as ps_chunk_step: nothing happens when ctrl->skip is set (the
 * reference neither tests these gradients for overflow nor restores these
 * parameters, fp16_cpu_adam.py:301-302, 485-486); otherwise every element gets
 * the update of ps_chunk_step with the gradient taken as fp32 (unscale by the
 * slot's loss scale, fp32 clamp when clipping is on, no world-size division).
 * 28 B/element.  The table is given in HOST memory, because the gradient
 * pointers change every step; it is validated, copied (the caller may reuse it
 * as soon as the call returns) and uploaded into table_dev, n_tensors rows of
 * device memory owned by the caller.  No synchronisation. */
int ps_tensor_table_step(const ps_tensor_desc* tensors_host, uint32_t n_tensors, uint32_t n_slots,
                         ps_tensor_desc* table_dev, const ps_step_ctrl* ctrl_dev, void* stream);

/* The multi-GPU chunk step as ONE kernel: the step of ps_chunk_step fused with
 * the reduce-scatter of the fp16 grad chunks before it
 * (patrickstar/core/client.py:818-856) and the all-gather of the fp16 param
 * chunks after it (client.py:428-497), over NVSwitch multicast memory.  Every
 * rank holds the whole fp16 chunk list in a buffer that is mapped into one
 * multicast object (same offset on every rank): fp16_local_base is this rank's
 * buffer, fp16_multicast_base the multicast mapping of it.  The chunk table
 * holds this rank's OWN chunks with h16 pointing into the local buffer.  For
 * each owned element the gradient is loaded as the switch-side sum over all
 * ranks' buffers (fp32 accumulation, one rounding to fp16) and the updated fp16
 * param is stored to all ranks' buffers (single elements at ragged ends and
 * segment boundaries go through peer_bases_dev, a device array of every rank's
 * buffer base, because there is no 16-bit multicast access).  ctrl's slots must carry
 * grad_divisor = world size (client.py:838).  The caller guarantees, with a
 * barrier across ranks on each side, that every rank's gradients are complete
 * before any rank launches and that no rank reads params or writes new
 * gradients before every rank's launch has finished. */
int ps_chunk_step_fused(const ps_chunk_desc* chunks_dev, uint32_t n_chunks, uint32_t max_numel,
                        const ps_segment* segs_dev, const ps_step_ctrl* ctrl_dev,
                        const void* fp16_local_base, const void* fp16_multicast_base,
                        const uint64_t* peer_bases_dev, int world_size, void* stream);

/* The same fusion over plain peer mappings (no multicast object): the gradient
 * of an owned element is the sum of the world_size ranks' values read through
 * peer_bases_dev, accumulated in fp32 in rank order and rounded once to fp16;
 * the updated fp16 param is stored into every rank's buffer.  world_size <= 8.
 * Same barriers as ps_chunk_step_fused. */
int ps_chunk_step_p2p(const ps_chunk_desc* chunks_dev, uint32_t n_chunks, uint32_t max_numel,
                      const ps_segment* segs_dev, const ps_step_ctrl* ctrl_dev, const void* fp16_local_base,
                      const uint64_t* peer_bases_dev, int world_size, void* stream);

/* ps_chunk_step_fused as a two-stage pipeline over the same multicast memory,
 * for measurements of how the NVLink round trip is best hidden: per owned chunk
 * a light kernel on the pipeline's own stream pulls the switch-side sum of the
 * gradients (multimem.ld_reduce) into one of two local staging buffers while
 * the step kernel on `stream` updates the previous chunk from its staging
 * buffer and stores the fp16 params to all ranks (multimem.st).  staging_dev:
 * 2 * max_numel fp16 elements of plain device memory owned by the caller.
 * Results are bit-identical to ps_chunk_step_fused.  ps_fused_pipe_create makes
 * the stream and events (no device memory). */
int ps_fused_pipe_create(void** pipe_out);
int ps_fused_pipe_destroy(void* pipe);
int ps_chunk_step_fused_staged(void* pipe, const ps_chunk_desc* chunks_dev, uint32_t n_chunks,
                               uint32_t max_numel, const ps_segment* segs_dev, const ps_step_ctrl* ctrl_dev,
                               const void* fp16_local_base, const void* fp16_multicast_base,
                               const uint64_t* peer_bases_dev, int world_size, uint16_t* staging_dev,
                               void* stream);

#define PS_COPY_MAX_CHUNKS 4096u /* owned chunks per ps_chunk_step_copy call */

/* The same multi-GPU step with the NVLink traffic handed to the copy engines,
 * pipelined chunk by chunk over plain peer mappings: while the step kernel works
 * on owned chunk k, the copy engines pull every peer's gradients of chunk k+1
 * into local staging buffers (the reduce-scatter's traffic) and push the updated
 * fp16 params of chunk k-1 into every peer's buffer (the all-gather's).  The
 * kernel sums the own slot and the staged copies in rank order in fp32 and
 * rounds once, exactly as ps_chunk_step_p2p does, so the two give identical
 * bits; it touches local memory only.  NVLink bytes per direction, rank and
 * group: 2 * (world_size - 1) chunks, at the copy engines' rate.
 *   chunks_host       : host copy of the chunk table (the copies need the fp16
 *                       addresses on the host)
 *   peer_bases_host   : every rank's fp16 buffer base as mapped on this rank
 *                       (world_size entries, entry `rank` = fp16_local_base)
 *   peer_bases_dev    : NULL, or the same array in device memory: the kernel then
 *                       stores the fp16 params into every rank's buffer itself
 *                       (posted peer stores) and the copy engines only pull
 *   staging_dev       : n_slots * (world_size - 1) * max_numel fp16 elements
 *                       (rounded up to a multiple of 8 per chunk copy), plain
 *                       device memory; more slots let the pulls run further ahead
 *   gather_table_dev  : n_chunks * world_size uint64 of device scratch
 * ps_copy_pipe_create makes the streams and events for n_slots (2..8) staging
 * slots (no device memory).  Same barriers across ranks as ps_chunk_step_fused;
 * world_size <= 8. */
int ps_copy_pipe_create(void** pipe_out, int n_slots);
int ps_copy_pipe_destroy(void* pipe);
int ps_chunk_step_copy(void* pipe, const ps_chunk_desc* chunks_dev, const ps_chunk_desc* chunks_host,
                       uint32_t n_chunks, uint32_t max_numel, const ps_segment* segs_dev,
                       const ps_step_ctrl* ctrl_dev, const void* fp16_local_base, const uint64_t* peer_bases_host,
                       const uint64_t* peer_bases_dev, int rank, int world_size, uint16_t* staging_dev,
                       uint64_t* gather_table_dev, void* stream);

/* dst[i] = the reduced gradient ps_chunk_step_p2p loads for the element at
 * fp16_local_ptr + 2*i of this rank's buffer.  For tests. */
int ps_p2p_reduce_probe(const void* fp16_local_ptr, const void* fp16_local_base, const uint64_t* peer_bases_dev,
                        int world_size, uint16_t* dst_dev, size_t n, void* stream);

/* dst[i] = switch-side sum over all ranks of the fp16 value at multicast
 * address fp16_multicast_ptr + 2*i — exactly what ps_chunk_step_fused loads as
 * the reduced gradient (n even, 16-byte aligned pointers).  For tests. */
int ps_multimem_reduce_probe(const void* fp16_multicast_ptr, uint16_t* dst_dev, size_t n, void* stream);

/* Copies the device scaler state / control block to the host.  Synchronises
 * `stream`.  (DynamicLossScaler.loss_scale, state["step"].) */
int ps_scaler_read(const ps_scaler_state* scaler_dev, ps_scaler_state* out_host, void* stream);
int ps_ctrl_read(const ps_step_ctrl* ctrl_dev, ps_step_ctrl* out_host, void* stream);

/* scaled = loss * cur_scale on the device (DynamicLossScaler.backward,
 * loss_scaler.py:188-190) without reading the scale back: fp32 in/out, n values. */
int ps_scale_loss(const float* loss_dev, float* out_dev, size_t n, const ps_scaler_state* scaler_dev,
                  void* stream);

/* ------------------------------------------------------------------ */
/* offload tier                                                         */
/* ------------------------------------------------------------------ */
#define PS_OFFLOAD_MAX_SLOTS 8

/* One piece of an offloaded local chunk: `numel` consecutive elements of its
 * fp32 master / momentum / variance in PINNED host memory (what the reference
 * keeps as CPU chunks under hybrid placement,
 * patrickstar/ops/fp16_cpu_adam.py:523-528, patrickstar/core/chunk_data.py:275-366)
 * and the index of the piece's descriptor in the device chunk table.  That
 * descriptor covers [first, first + numel) of the chunk (ps_chunk_desc.reserved
 * = first, .numel = first + numel) and its p32 / exp_avg / exp_avg_sq point
 * `first` elements BEFORE the staging slot (i % n_slots) that the i-th piece of
 * a ps_offload_step call uses, so that chunk-local indices address the slot;
 * h16 and the segment range are the chunk's own.  Pieces smaller than a chunk
 * shorten the fill and drain of the pipeline. */
typedef struct ps_offload_chunk {
    float* p32_host;
    float* exp_avg_host;
    float* exp_avg_sq_host;
    uint32_t numel;
    uint32_t desc_index;
} ps_offload_chunk;

/* Creates the pipeline object: three side streams and 3 * n_slots + 1 events on
 * the current device.  No device memory is allocated; the caller owns the
 * staging slots.  n_slots = 2 is double buffering. */
int ps_offload_create(void** pipeline_out, int n_slots);
int ps_offload_destroy(void* pipeline);

/* Streams n_chunks offloaded chunks through the staging slots around the fused
 * chunk step, replacing the reference's synchronous chunk moves and CPU Adam
 * for host-resident chunks (patrickstar/ops/chunk_io_buff.py:116-126, 241-247).
 * staging_dev[3*s .. 3*s+2] = p32 / exp_avg / exp_avg_sq buffers of slot s, each
 * at least numel floats.  Must be called after ps_step_begin on `stream`; the
 * copies and kernels run on the pipeline's own streams, overlapped with whatever
 * the caller enqueues on `stream` next, and `stream` is made to wait for the
 * last write-back before the call returns (no host synchronisation). */
int ps_offload_step(void* pipeline, const ps_offload_chunk* chunks_host, uint32_t n_chunks,
                    float* const* staging_dev, const ps_chunk_desc* chunks_dev,
                    const ps_segment* segs_dev, const ps_step_ctrl* ctrl_dev, void* stream);
int ps_offload_last_cuda_error(void);

/* ------------------------------------------------------------------ */
/* allocation-free variant                                              */
/* ------------------------------------------------------------------ */
#define PS_STATIC_MAX_CHUNKS 256u    /* chunk descriptors per call   */
#define PS_STATIC_MAX_SEGMENTS 4096u /* segments per call            */

/* No counterpart in the reference.  The same fused chunk step as
 * ps_chunk_step, for callers that cannot call cudaMalloc: a host that has
 * handed the whole GPU to its own pool and budgets every byte of it (the way
 * PatrickStar's chunk manager and memory tracer do), or code on a latency
 * path where cudaMalloc's device-wide synchronisation is not acceptable.  Such
 * a caller has nowhere to put the device-side chunk table, segment table and
 * control block that ps_chunk_step reads.  Here all three are taken from host
 * memory and staged into a fixed array that lives inside the library's device
 * image (about 81 KB on every GPU that loads the library, held until the
 * process exits).  Nothing is allocated or freed, by this library or through
 * any other.
 *
 *   chunks_host / segs_host : the tables of ps_chunk_step, in host memory; the
 *                             pointers inside ps_chunk_desc are device
 *                             addresses of the caller's chunks as before
 *   slots_host[n_slots]     : the per-slot constants ps_step_begin would have
 *                             prepared (n_slots <= PS_MAX_SLOTS)
 *   skip                    : non-zero = restore the fp16 slots from the fp32
 *                             master instead of updating
 *
 * Limits: n_chunks <= PS_STATIC_MAX_CHUNKS and n_segs <= PS_STATIC_MAX_SEGMENTS,
 * else PS_ERR_LIMIT and nothing is enqueued; larger jobs are split by the
 * caller.  The tables are validated like ps_table_check does, and
 * ps_chunk_desc.reserved must be 0 here (PS_ERR_TABLE otherwise).
 *
 * The first call on each device looks up the array's device address
 * (cudaGetSymbolAddress); make that first call before any stream capture.
 * All calls share the one array and each call overwrites it completely:
 * calls on one stream are ordered and safe, calls that can overlap on the GPU
 * (different streams, different threads) race on it and must be serialised by
 * the caller.
 *
 * The host tables and slots are copied, before the call returns, into a
 * pageable host buffer the library keeps per calling thread, and uploaded from
 * there; the caller's own tables — pageable, pinned or registered — may
 * therefore be changed or freed as soon as the call returns. */
int ps_chunk_step_static(const ps_chunk_desc* chunks_host, uint32_t n_chunks, uint32_t max_numel,
                         const ps_segment* segs_host, uint32_t n_segs,
                         const ps_hyper_slot* slots_host, uint32_t n_slots, int skip, void* stream);

/* Tuning knobs for measurements: "unroll" (1, 2, 4: 128-bit groups per thread
 * per tile of the step kernels), "scan_unroll" (1, 2, 4), "blocks_per_sm"
 * (0 = occupancy calculator), "bulk" (0, or 2..4 stages of the bulk-async
 * staged chunk step), "fused_depth" (2, 4, 8: reduced-gradient loads a thread
 * of ps_chunk_step_fused keeps in flight), "fused_min_blocks" / "p2p_min_blocks"
 * (2..4: resident CTAs per SM the fused kernels' register budget is cut for),
 * "fused_blocks_per_sm", "pull_blocks_per_sm" / "staged_blocks_per_sm" (grids of
 * the two kernels of ps_chunk_step_fused_staged), "p2p_unroll" (0 = by world
 * size, 1, 2), "p2p_blocks_per_sm".  The defaults are the measured best; no
 * counterpart in the reference. */
int ps_tune(const char* key, int value);

/* Kernel launch counter: number of kernels this library has launched in this
 * process (for benchmark bookkeeping). */
uint64_t ps_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* PS_B200_H */
