/*
 * libsynaptik_cuda.so -- C ABI of the B200 (sm_100a) CUDA backend for Synaptik.
 *
 * The shape follows the one native boundary the reference ships, the Metal foundation library
 * ("ABI version 7", modules/backend/metal/macos-arm64/README.md: thirteen exported symbols,
 * opaque void* handle families, int32 status returns, created handles through caller-supplied
 * output cells that stay NULL on failure, unsigned 64-bit sizes and offsets).  A Java binding
 * reaches these symbols through java.lang.foreign downcalls exactly as
 * modules/backend/metal/.../MetalNativeApi.java:3648-3708 binds the Metal ones.
 *
 * Every function except synaptik_cuda_abi_version returns a status (0 = success).  No function
 * aborts the process, resets a device, or falls back to a CPU implementation: without a usable
 * CUDA device context_create returns SYNAPTIK_CUDA_STATUS_NO_DEVICE and nothing else can run.
 * Entry points are thread-safe per handle; work is issued on the owning context's stream and
 * every call that hands results to the host returns only after they are usable.
 */
#ifndef SYNAPTIK_CUDA_H
#define SYNAPTIK_CUDA_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SYNAPTIK_CUDA_ABI_VERSION 1u

#if defined(__GNUC__)
#define SYNAPTIK_CUDA_API __attribute__((visibility("default")))
#else
#define SYNAPTIK_CUDA_API
#endif

/* Status values 0..13 keep the numeric meaning of the Metal library's table
 * (modules/backend/metal/macos-arm64/README.md, "Status values"); 14 and 15 are new. */
enum {
    SYNAPTIK_CUDA_STATUS_OK = 0,
    SYNAPTIK_CUDA_STATUS_INVALID_ARGUMENT = 1,
    SYNAPTIK_CUDA_STATUS_NO_DEVICE = 2,
    SYNAPTIK_CUDA_STATUS_NO_STREAM = 3,            /* Metal: NO_COMMAND_QUEUE */
    SYNAPTIK_CUDA_STATUS_ALLOCATION_FAILED = 4,
    SYNAPTIK_CUDA_STATUS_RANGE_OUT_OF_BOUNDS = 5,  /* copy outside a buffer, or a label outside [0, classes) */
    SYNAPTIK_CUDA_STATUS_COPY_FAILED = 6,
    SYNAPTIK_CUDA_STATUS_INTERNAL_ERROR = 7,
    SYNAPTIK_CUDA_STATUS_UNSUPPORTED_SHAPE = 8,
    SYNAPTIK_CUDA_STATUS_GRAPH_COMPILATION_FAILED = 9,  /* malformed program image */
    SYNAPTIK_CUDA_STATUS_INCOMPATIBLE_RESOURCE = 10,    /* wrong context, wrong extent, aliasing */
    SYNAPTIK_CUDA_STATUS_EXECUTION_FAILED = 11,         /* CUDA error, or a non-finite optimizer intermediate */
    SYNAPTIK_CUDA_STATUS_KERNEL_COMPILATION_FAILED = 12,
    SYNAPTIK_CUDA_STATUS_UNSUPPORTED_OPERATION = 13,    /* valid image, operation outside capability */
    SYNAPTIK_CUDA_STATUS_TIMEOUT = 14,                  /* a bounded device-side wait expired */
    SYNAPTIK_CUDA_STATUS_COMM_FAILED = 15               /* NCCL unavailable or a collective failed */
};

/* Replaces synaptik_metal_foundation_abi_version (README.md "ABI version 7"); the Java side
 * probes it first and refuses a mismatch (MetalNativeApi.java:3648-3708). */
SYNAPTIK_CUDA_API uint32_t synaptik_cuda_abi_version(void);

/* ---- context: replaces synaptik_metal_context_create / _release ------------------------------
 * One context per GPU ordinal: a compute stream, a communication stream and the scratch arena
 * of the tensor-core GEMM path.  (MetalDeviceContext.java:123-216 is the Java owner.) */
SYNAPTIK_CUDA_API int32_t synaptik_cuda_context_create(int32_t device_ordinal, void **out_context);
SYNAPTIK_CUDA_API int32_t synaptik_cuda_context_release(void *context);
/* Named integer options.  "gemm_engine": 0 = automatic (tensor cores for large products, exact
 * sequential CUDA-core kernel for small ones), 1 = always the exact CUDA-core kernel,
 * 2 = tensor cores whenever the shape allows.  "time_steps": 1 = bracket every step of later runs
 * with CUDA events (see synaptik_cuda_executable_step_timings).  "fused_planes": whether a GEMM whose
 * result a later GEMM reads writes that operand's hi / lo planes from its own epilogue instead of leaving
 * them to a separate pass; 0 = never, 1 (default) = where it pays (two-SM products, whose write-out goes
 * through shared memory and TMA stores, and one-accumulator products with K >= 2048), 2 = every product
 * with K >= 2048, 3 = every product.  Results do not depend on it.  "gemm_promote": 1 (default) = the
 * tensor-core GEMM keeps only short partial sums (256 or 512 contraction steps) in tensor memory and
 * adds them into round-to-nearest FP32 register sums; 0 = one tensor-memory accumulator over the
 * whole contraction (faster epilogue, error grows with K).  "gemm_chunk": contraction steps per
 * tensor-memory partial sum of executables created afterwards, a multiple of 32, 0 (default) = 512 (256
 * from K = 8192 on); shorter partial sums are more exact and slower (128: a quarter of the error, about
 * 6 % more time on the 4096-wide layers).  "gemm_pair": 1 (default) = products with
 * at least 256 rows use two-SM tiles (clusters of two blocks, tcgen05 cta_group::2); 0 = one-SM tiles
 * only.  "gemm_slices": 1 (default) = a two-SM product without epilogue work (a weight gradient) may
 * split its contraction into up to four slices when that shortens the last wave of the persistent
 * grid; the slices' partial products are added in ascending order by a second kernel; 0 = never;
 * 2 = also cut a product of one wave or less into at least two slices, so that it has units to spare
 * when another kernel (an all-reduce) holds some SMs.
 * "gemm_dynamic": 1 (default) = executables created afterwards let the two-SM kernel's block pairs take
 * their tiles one by one from a counter, so a pair whose SMs were held by another kernel (an
 * all-reduce on the communication stream) just takes fewer tiles; 0 = fixed round-robin assignment.
 * The result does not depend on the assignment.  "comm_timeout_ms" (default 30000): how
 * long the host waits, in any call that returns results, for work that has a collective in front of it
 * before it gives up, aborts the communicator and returns COMM_FAILED.  Unknown names return
 * INVALID_ARGUMENT. */
SYNAPTIK_CUDA_API int32_t synaptik_cuda_context_set_option(void *context, const char *name, int64_t value);
/* Blocks until all work issued on the context has finished. */
SYNAPTIK_CUDA_API int32_t synaptik_cuda_context_synchronize(void *context);
/* CUDA-event stopwatch on the context's compute stream (the stream every kernel of the context is
 * launched on): start records an event, stop records another, waits for it and returns the device
 * time between the two in milliseconds. */
SYNAPTIK_CUDA_API int32_t synaptik_cuda_context_timer_start(void *context);
SYNAPTIK_CUDA_API int32_t synaptik_cuda_context_timer_stop(void *context, double *out_milliseconds);
/* Self-test of the bounded device-side waits (no counterpart in the reference).  Every wait inside the
 * tensor-core GEMM kernels gives up after two seconds instead of spinning forever; the kernel then
 * leaves in an orderly way and the run returns TIMEOUT.  This call launches one 32-thread block that
 * runs the same wait routine on a barrier which nothing ever signals, with a limit of
 * `limit_microseconds` (1 .. 2000000), and reports the outcome like a run would: it returns
 * SYNAPTIK_CUDA_STATUS_TIMEOUT, never OK, and the context is as usable afterwards as before. */
SYNAPTIK_CUDA_API int32_t synaptik_cuda_context_wait_probe(void *context, uint64_t limit_microseconds);
/* Measurement and test instrument (no counterpart in the reference): enqueues, on the context's
 * communication stream, `blocks` thread blocks (0 .. the SM count) that each hold one SM for
 * `hold_microseconds` (at most 100000) and then end by themselves, the way the blocks of an all-reduce
 * hold SMs while the backward pass runs.  Returns at once.  With it one GPU shows how the tensor-core
 * products give way to a co-tenant: their results must not change, only their duration. */
SYNAPTIK_CUDA_API int32_t synaptik_cuda_context_occupy(void *context, int32_t blocks, uint64_t hold_microseconds);

/* ---- buffers: replace synaptik_metal_buffer_create / _release / _upload / _download ----------
 * Device-resident linear memory.  upload/download move raw little-endian element bytes and
 * return when the copy is complete; the *_canonical forms take or produce the engine's
 * canonical BIG-ENDIAN element bytes (modules/model/.../HostTensorValue.java:108-110,
 * EngineBackendComposition.copyToCanonicalHostBytes :153) by swapping element_bytes-wide
 * groups on the host side of the copy (element_bytes in {1,2,4,8}). */
SYNAPTIK_CUDA_API int32_t synaptik_cuda_buffer_create(void *context, uint64_t bytes, void **out_buffer);
SYNAPTIK_CUDA_API int32_t synaptik_cuda_buffer_release(void *buffer);
SYNAPTIK_CUDA_API int32_t synaptik_cuda_buffer_upload(void *buffer, uint64_t offset, const void *source, uint64_t bytes);
SYNAPTIK_CUDA_API int32_t synaptik_cuda_buffer_download(void *buffer, uint64_t offset, void *destination, uint64_t bytes);
SYNAPTIK_CUDA_API int32_t synaptik_cuda_buffer_upload_canonical(void *buffer, uint64_t offset, const void *source,
                                              uint64_t bytes, uint32_t element_bytes);
SYNAPTIK_CUDA_API int32_t synaptik_cuda_buffer_download_canonical(void *buffer, uint64_t offset, void *destination,
                                                uint64_t bytes, uint32_t element_bytes);
/* Asynchronous forms for callers that keep pinned host memory: they enqueue on the context's
 * stream and return at once; synaptik_cuda_context_synchronize orders the host after them. */
SYNAPTIK_CUDA_API int32_t synaptik_cuda_buffer_upload_async(void *buffer, uint64_t offset, const void *source, uint64_t bytes);
SYNAPTIK_CUDA_API int32_t synaptik_cuda_buffer_download_async(void *buffer, uint64_t offset, void *destination, uint64_t bytes);
/* Upload from pinned host memory on the context's copy stream, concurrently with the work already
 * enqueued on the compute stream (a training loop fills the next batch's buffers while the current
 * step runs; no counterpart in the Metal ABI, whose memory is unified).  Ordering is by buffer: the
 * copy starts after every executable run enqueued so far that was bound to this buffer, and every
 * later run bound to it (and every later upload / download of it) starts after the copy.
 * synaptik_cuda_context_synchronize also waits for prefetches.  Optimizer steps are not tracked: do
 * not prefetch into a parameter or gradient buffer. */
SYNAPTIK_CUDA_API int32_t synaptik_cuda_buffer_prefetch(void *buffer, uint64_t offset, const void *source, uint64_t bytes);
/* Device address and size of a buffer, for callers that share it with other CUDA code. */
SYNAPTIK_CUDA_API int32_t synaptik_cuda_buffer_device_pointer(void *buffer, uint64_t *out_address, uint64_t *out_bytes);
/* Page-locked host memory for staging (EngineBackendComposition.borrow :118 uploads from it). */
SYNAPTIK_CUDA_API int32_t synaptik_cuda_host_alloc(uint64_t bytes, void **out_pointer);
SYNAPTIK_CUDA_API int32_t synaptik_cuda_host_free(void *pointer);

/* ---- prepared executables: replace synaptik_metal_mpsgraph_executable_create/_release/_run --
 * `program` is one little-endian "SCU1" image (layout in synaptik_b200/csrc/program.hpp) that
 * lists a whole backend partition in topological order: value descriptors (dtype, shape,
 * element strides, role), nodes (operation wire code, attributes, input and output value
 * references), the ordered feed values and the ordered publication values.  Creation validates
 * the image, lowers it to fused kernel launches and reserves every intermediate; it performs no
 * device work on the hot path.  run binds `input_count` buffers to the feeds and `output_count`
 * buffers to the publications in image order (the role BoundInvocation.executeBound plays,
 * modules/runtime/.../execution/PreparedExecutable.java:254,421) and returns when the
 * publications are complete in device memory. */
SYNAPTIK_CUDA_API int32_t synaptik_cuda_executable_create(void *context, const uint8_t *program, uint32_t program_bytes,
                                        void **out_executable);
SYNAPTIK_CUDA_API int32_t synaptik_cuda_executable_release(void *executable);
SYNAPTIK_CUDA_API int32_t synaptik_cuda_executable_run(void *executable, int32_t input_count, void *const *inputs,
                                     int32_t output_count, void *const *outputs);
/* Same binding, but only enqueues the launches and returns; device-side failures (label range,
 * bounded-wait expiry) are then reported by the next synaptik_cuda_executable_finish. */
SYNAPTIK_CUDA_API int32_t synaptik_cuda_executable_enqueue(void *executable, int32_t input_count, void *const *inputs,
                                         int32_t output_count, void *const *outputs);
SYNAPTIK_CUDA_API int32_t synaptik_cuda_executable_finish(void *executable);
/* Writes a NUL-terminated, line-per-launch description of the lowered plan (kernel, shapes,
 * engine) into `text`; needs no GPU and is what the host-logic tests read.  With a NULL context
 * the image is lowered for a default device description.  Returns INVALID_ARGUMENT when
 * capacity is too small (required size, including the NUL, is stored in *out_required). */
SYNAPTIK_CUDA_API int32_t synaptik_cuda_program_describe(const uint8_t *program, uint32_t program_bytes, char *text,
                                       uint64_t capacity, uint64_t *out_required);
/* Device time in milliseconds of the most recent finished run (CUDA events on the context
 * stream); the hook for trace payloads (modules/trace BackendInvocationOutcome). */
SYNAPTIK_CUDA_API int32_t synaptik_cuda_executable_last_timing(void *executable, double *out_milliseconds);
/* The plan of this executable (as lowered under its context's options), one line per step, in
 * the format of synaptik_cuda_program_describe. */
SYNAPTIK_CUDA_API int32_t synaptik_cuda_executable_describe(void *executable, char *text, uint64_t capacity, uint64_t *out_required);
/* With the context option "time_steps" = 1, every step of a run is bracketed by CUDA events (a
 * tensor-core GEMM step brackets the GEMM kernel alone, not the operand split).  This call waits
 * for the most recent run and stores one duration in milliseconds per plan step, in plan order;
 * the number of steps is stored in *out_count. */
SYNAPTIK_CUDA_API int32_t synaptik_cuda_executable_step_timings(void *executable, double *out_milliseconds, uint64_t capacity,
                                                              uint64_t *out_count);
/* Number of kernel launches the most recent run issued. */
SYNAPTIK_CUDA_API int32_t synaptik_cuda_executable_launch_count(void *executable, uint64_t *out_launches);

/* ---- training bridge: device-resident optimizer ----------------------------------------------
 * Replaces the host loops TrainingParameter.stageUpdate32 (SGD, modules/training/.../
 * TrainingParameter.java:622-672) and stageAdaptive32 / stageAdaptiveElement32 (Adam, AdamW,
 * :433-525) with one fused pass over all parameters.  Hyper-parameters arrive as doubles and are
 * narrowed to binary32 first, as AdaptiveCoefficients.forParameter does (:33-58).  Moments live
 * in device buffers owned by the optimizer handle.
 *   kind 0 = SGD   : hyper = {learning_rate, momentum, dampening, weight_decay, nesterov(0/1)}
 *   kind 1 = Adam  : hyper = {learning_rate, beta1, beta2, epsilon, weight_decay}
 *   kind 2 = AdamW : same five values, decoupled decay
 * step applies one update with gradients[i] matching parameters[i] element for element.
 *
 * A step is a transaction, like the reference's stage / validate / commit
 * (modules/training/.../TrainingSession.java:1151-1171, TrainingParameter.java:391-409).  When any
 * intermediate of the update is non-finite the step returns EXECUTION_FAILED, and when the run whose
 * gradients it consumes had already failed on the device (a label outside [0, classes): status 5; a
 * bounded wait that expired: 14; a collective that was given up: 15) it returns that status; in both
 * cases parameters, moments, the pending gradient sum, the step count and the count of accumulated
 * runs are bit for bit what they were before the call.  The update kernels write candidates into a
 * second set of arrays and the handle exchanges the two sets, so creating an optimizer allocates one
 * more array per parameter and per moment, and the device address of a parameter buffer
 * (synaptik_cuda_buffer_device_pointer) changes with every step; bytes of a parameter buffer past
 * element_counts[i] elements are not carried from step to step.  With the *_enqueue forms the verdict
 * arrives with the next *_finish of the context (optimizer or executable): a failure voids the failed
 * step and every step enqueued after it, and synaptik_cuda_optimizer_steps counts enqueued steps
 * until then. */
SYNAPTIK_CUDA_API int32_t synaptik_cuda_optimizer_create(void *context, int32_t kind, const double *hyper, int32_t hyper_count,
                                       int32_t parameter_count, void *const *parameters,
                                       const uint64_t *element_counts, void **out_optimizer);
SYNAPTIK_CUDA_API int32_t synaptik_cuda_optimizer_release(void *optimizer);
SYNAPTIK_CUDA_API int32_t synaptik_cuda_optimizer_step(void *optimizer, int32_t gradient_count, void *const *gradients);
/* Enqueue-only form; the non-finite flag is then reported by synaptik_cuda_optimizer_finish. */
SYNAPTIK_CUDA_API int32_t synaptik_cuda_optimizer_step_enqueue(void *optimizer, int32_t gradient_count, void *const *gradients);
SYNAPTIK_CUDA_API int32_t synaptik_cuda_optimizer_finish(void *optimizer);
/* Gradient modes of one training run (modules/training/.../GradientMode.java:4-22 as applied by
 * TrainingSession.java:583-640).  RESET_AND_STEP (0): update from this run's gradients, drop any
 * pending sum.  ACCUMULATE (1): pending = pending + gradient (one binary32 addition per element,
 * TrainingParameter.java:373-390); parameters, moments and the step count do not change.
 * ACCUMULATE_AND_STEP (2): update from pending + gradient, then clear the pending sum.  A non-finite
 * sum reports status 11 like any other non-finite intermediate and leaves the pending sum as it was.  zero_grad clears the pending sum
 * (TrainingSession.zeroGrad, :640-652); accumulated_runs counts the runs in it. */
enum { SYNAPTIK_CUDA_GRADIENT_RESET_AND_STEP = 0, SYNAPTIK_CUDA_GRADIENT_ACCUMULATE = 1, SYNAPTIK_CUDA_GRADIENT_ACCUMULATE_AND_STEP = 2 };
SYNAPTIK_CUDA_API int32_t synaptik_cuda_optimizer_run(void *optimizer, int32_t gradient_mode, int32_t gradient_count, void *const *gradients);
SYNAPTIK_CUDA_API int32_t synaptik_cuda_optimizer_run_enqueue(void *optimizer, int32_t gradient_mode, int32_t gradient_count, void *const *gradients);
SYNAPTIK_CUDA_API int32_t synaptik_cuda_optimizer_zero_grad(void *optimizer);
SYNAPTIK_CUDA_API int32_t synaptik_cuda_optimizer_accumulated_runs(void *optimizer, uint64_t *out_runs);
/* Completed optimizer steps, and copies of one parameter's optimizer-width arrays for TrainingState
 * snapshots and restores (TrainingParameter.java:894-941, :1000-1060): slot 0 = momentum / first
 * moment, 1 = second moment, 2 = pending gradient sum.  The plain forms move raw little-endian
 * binary32; the _canonical forms move the big-endian element bytes the snapshot stores.
 * set_progress restores the two counters of a snapshot. */
SYNAPTIK_CUDA_API int32_t synaptik_cuda_optimizer_steps(void *optimizer, uint64_t *out_steps);
SYNAPTIK_CUDA_API int32_t synaptik_cuda_optimizer_download_state(void *optimizer, int32_t parameter_index, int32_t slot,
                                               void *destination, uint64_t bytes);
SYNAPTIK_CUDA_API int32_t synaptik_cuda_optimizer_upload_state(void *optimizer, int32_t parameter_index, int32_t slot,
                                             const void *source, uint64_t bytes, uint64_t completed_steps);
SYNAPTIK_CUDA_API int32_t synaptik_cuda_optimizer_download_state_canonical(void *optimizer, int32_t parameter_index, int32_t slot,
                                                         void *destination, uint64_t bytes);
SYNAPTIK_CUDA_API int32_t synaptik_cuda_optimizer_upload_state_canonical(void *optimizer, int32_t parameter_index, int32_t slot,
                                                       const void *source, uint64_t bytes);
SYNAPTIK_CUDA_API int32_t synaptik_cuda_optimizer_set_progress(void *optimizer, uint64_t completed_steps, uint64_t accumulated_runs);

/* ---- data-parallel communicator (no counterpart in the reference, which is single-device) ----
 * One rank per process and GPU.  unique_id is the 128-byte NCCL id produced by
 * synaptik_cuda_comm_unique_id on rank 0 and distributed by the caller.  An executable with an
 * attached communicator sum-allreduces the listed publications (gradients) on the context's
 * communication stream as soon as each is final, overlapping the rest of the backward pass, and
 * run/finish return after the reductions.  attach_comm refuses (INCOMPATIBLE_RESOURCE) a publication
 * that a later step of the same executable still reads.  It waits for the executable's runs in flight and
 * plans tensor-core products of at most one tile per SM pair again with their contraction in slices (see
 * "gemm_slices"), because a single wave of tiles cannot give way to the collective's blocks; such a product's
 * sums then round differently than without a communicator, within the same bound.  The host never waits for a collective without
 * a limit: finish, run and comm_allreduce_sum_f32 poll NCCL's asynchronous error state and, after the
 * context option "comm_timeout_ms", mark the steps in flight as failed, abort the communicator and
 * return COMM_FAILED; the communicator is unusable from then on (every call on it returns
 * COMM_FAILED), the context and its buffers are not.  The environment variable
 * SYNAPTIK_NCCL_LIBRARY names the NCCL library file to bind; when it is set and the file does not
 * load, the communicator calls return COMM_FAILED (no other copy is looked for). */
SYNAPTIK_CUDA_API int32_t synaptik_cuda_comm_unique_id(uint8_t *out_id128);
SYNAPTIK_CUDA_API int32_t synaptik_cuda_comm_create(void *context, int32_t world_size, int32_t rank, const uint8_t *unique_id128,
                                  void **out_comm);
SYNAPTIK_CUDA_API int32_t synaptik_cuda_comm_release(void *comm);
SYNAPTIK_CUDA_API int32_t synaptik_cuda_comm_allreduce_sum_f32(void *comm, void *buffer, uint64_t offset, uint64_t element_count);
SYNAPTIK_CUDA_API int32_t synaptik_cuda_executable_attach_comm(void *executable, void *comm, int32_t output_count,
                                             const int32_t *output_indices);

/* ---- column sums for callers that must not allocate (no counterpart in the reference) ---------
 * Some callers hold a device context in which allocation is off limits: code running inside a
 * memory-pool or capture-sensitive region of a host framework, a plugin that was handed fixed
 * buffers by its owner, a real-time loop that may not touch the allocator.  For them this one
 * entry point computes out[n] = sum over rows of in[row, n] (the bias gradient, FP32 in and out,
 * binary64 accumulation, fixed summation order) exactly like the SUM_TO_SHAPE step of an
 * executable, but keeps its intermediate partial sums in a 2 MiB array that is part of the library
 * image on every GPU that loads it, and calls no allocating routine of CUDA or of any library.
 *   - `input` holds rows x cols dense row-major floats at byte offset 0, `output` at least cols
 *     floats; both are buffers of `context`.
 *   - Shapes whose partial sums do not fit the array (more than 262144 of them) are refused with
 *     UNSUPPORTED_SHAPE: every shape of at most 131072 columns fits, none above 262144 columns
 *     does, in between it depends on the row count.
 *   - The first call on a device looks up the array's device address; make that first call
 *     outside any stream capture.
 *   - All calls on a device share the one array.  A call overwrites every partial it later reads,
 *     so nothing is left over from the previous call, but two calls whose kernels overlap on the
 *     GPU (different contexts or streams) would race on it: serialise them.
 * The work is enqueued on the context's stream and the call returns after it has finished. */
SYNAPTIK_CUDA_API int32_t synaptik_cuda_column_sums_no_alloc(void *context, void *input, uint64_t rows, uint64_t cols, void *output);

#ifdef __cplusplus
}
#endif
#endif
