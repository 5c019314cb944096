/*
 * ayla_b200 -- C ABI of the sm_100a (B200) GEMM backend.
 *
 * Every entry point is plain C: raw device pointers, sizes, an opaque stream
 * handle.  The library never allocates or frees device memory and never
 * synchronises: a call enqueues its kernel on the given stream and returns.
 * All functions return 0 on success or one of the AYLA_B200_E_* codes;
 * ayla_b200_last_error() then holds a thread-local message.
 *
 * Operand convention (same as the reference's ops, ayla/gemm_jit.py:267-307,
 * :396-411): all tensors are contiguous row-major 16-bit floats,
 *     mm     out[M,N]     = a[M,K]   @ bt[N,K]^T
 *     addmm  out[M,N]     = bias[N] + a[M,K] @ bt[N,K]^T      (bias added in fp32,
 *                                                             before the one rounding)
 *     bmm    out[B,M,N]   = a[B,M,K] @ bt[B,N,K]^T            (per batch)
 * with fp32 accumulation and a single round-to-nearest-even to the output type
 * (ayla/passes/lower_to_ptx_template.py:134-149).
 */
#ifndef AYLA_B200_H_
#define AYLA_B200_H_

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define AYLA_B200_API __attribute__((visibility("default")))
#else
#define AYLA_B200_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

#define AYLA_B200_OK 0
#define AYLA_B200_E_INVALID 1     /* bad argument (null pointer, non-positive extent, ...) */
#define AYLA_B200_E_UNSUPPORTED 2 /* shape/alignment/config outside what the kernels cover */
#define AYLA_B200_E_WORKSPACE 3   /* workspace missing or too small for the chosen config */
#define AYLA_B200_E_CUDA 4        /* a CUDA runtime/driver call failed */
#define AYLA_B200_E_NOT_INIT 5    /* ayla_b200_init() has not succeeded on this device */

#define AYLA_B200_OP_MM 0
#define AYLA_B200_OP_ADDMM 1
#define AYLA_B200_OP_BMM 2

#define AYLA_B200_F16 0
#define AYLA_B200_BF16 1

/*
 * One kernel schedule.  It is the sm_100a counterpart of the reference's
 * schedule dictionaries (keys of ayla/gemm_collection/gemm.py:179-198 as stored
 * in ayla/gemm_schedule_table.py:14): tile_n ~ output_n_tile, stages ~
 * operand_stages, grid_ctas ~ output_cta_count, group_m ~ the raster keys
 * (swap_output_grid_axes / output_tile_fast_axis), l2_hint_* ~
 * {lhs,rhs}_l2_cache_hint, cta_group ~ cluster_m_ctas.  The row tile is fixed
 * at 128 per CTA (256 per CTA pair).
 */
typedef struct ayla_b200_config {
  int32_t tile_n;    /* accumulator columns per tile: 16,32,64,128,192,256 (16/32 only with swap_ab, 192 only without) */
  int32_t cta_group; /* 1, or 2 = two CTAs share one 256-row tile */
  int32_t swap_ab;   /* 1 = compute out^T = bt @ a^T (rows of bt fill the 128-row tile); small M */
  int32_t split_k;   /* >= 1; > 1 needs a workspace */
  int32_t group_m;   /* raster: row tiles per group, >= 1 */
  int32_t grid_ctas; /* persistent grid size, 0 = one CTA per SM (capped by the work) */
  int32_t l2_hint_a; /* 0 normal, 1 evict_first, 2 evict_last; a/bt as passed by the caller */
  int32_t l2_hint_b;
  int32_t split_tail; /* wave quantisation: 1 = apply split_k only to the tiles of the last, partial
                         wave; 2 = do those tiles as two half-width units each (split_k must be 1) */
  int32_t l2_prefetch; /* k-blocks (of 64) the TMA producer prefetches into L2 ahead of its
                          shared-memory loads; 0 = off.  Measured slower on every shape tried so far;
                          kept as a tuning knob, never chosen by the default. */
  int32_t cluster_split; /* 1 = the split_k (2, 4 or 8) k-splits of a tile run as the CTAs (CTA
                            pairs when cta_group = 2) of one thread-block cluster and are
                            summed through distributed shared memory: no workspace, no global
                            round trip; split_k * cta_group <= 8 */
  int32_t stream_k;   /* 1 = stream-K schedule: every CTA takes an equal contiguous share of all
                         (tile, k-block) work; tiles cut between CTAs are reduced through the
                         workspace.  Excludes split_k > 1 and split_tail. */
  int32_t tile_rows;  /* swap_ab only: rows of bt per tile, 8..128 (0 = 128).  The MMA still spans
                         128 rows; fewer rows per tile means more, lighter tiles, so that a
                         weight whose 128-row tiles would leave SMs idle (112 tiles for
                         n = 14336 on 148 SMs) is streamed by all of them. */
  int32_t early_prefetch; /* k-blocks (0..32) of a CTA's first tile that its producer asks into L2 before
                             the kernel waits for the preceding launch in the stream (launch overlap on).
                             A prefetch delivers nothing into the kernel and L2 stays coherent with
                             whatever that launch still writes, so this is safe whatever it produces;
                             it fills the DRAM time the preceding launch's tail leaves idle.  Pays for
                             weight-streaming (small M) launches issued back to back, costs a little
                             where the operands are L2-resident anyway. */
} ayla_b200_config;

/*
 * Per-device set-up: opts every kernel into its shared-memory size and resolves
 * the driver's tensor-map encoder.  Call once per device before the first
 * launch and outside CUDA-graph capture.  Replaces the lazy module load of the
 * reference's launcher (ayla/ptx_runtime.py:358-369, :53-73).
 */
AYLA_B200_API int ayla_b200_init(int device);

/*
 * out = [bias +] a @ bt^T on `stream` (a cudaStream_t).  Replaces the kernel
 * launch behind gemm_op (ayla/gemm_jit.py:339-393 -> ayla/ptx_runtime.py:379-391,
 * :237-282).  `bias` is read only for AYLA_B200_OP_ADDMM; `batch` must be 1
 * unless op is AYLA_B200_OP_BMM.  Requirements: n % 8 == 0 and k % 8 == 0 (16-byte
 * row pitch for TMA), all pointers 16-byte aligned.  cfg == NULL picks a schedule
 * with ayla_b200_default_config.  `workspace` is needed only when the schedule has
 * split_k > 1; it must hold ayla_b200_workspace_bytes(...) bytes, the first
 * ayla_b200_workspace_counter_bytes(...) of them zero before the first use (the
 * kernel leaves them zero).  `status`, if non-NULL, is a uint32 the device can write
 * (device memory, or pinned host memory, which the host can then read without
 * synchronising); the kernel sets it to a non-zero code when one of its bounded
 * waits gives up; zero it first.
 */
AYLA_B200_API int ayla_b200_gemm(int op, int dtype, const void* bias, const void* a, const void* bt, void* out,
                   int64_t batch, int64_t m, int64_t n, int64_t k, const ayla_b200_config* cfg,
                   void* workspace, size_t workspace_bytes, uint32_t* status, void* stream);

/* Activations of ayla_b200_gemm_act. */
#define AYLA_B200_ACT_NONE 0
#define AYLA_B200_ACT_RELU 1
#define AYLA_B200_ACT_SIGMOID 2
#define AYLA_B200_ACT_SILU 3
#define AYLA_B200_ACT_GELU 4      /* 0.5 x (1 + erf(x / sqrt 2)) */
#define AYLA_B200_ACT_GELU_TANH 5 /* the tanh approximation */

/*
 * ayla_b200_gemm with an activation fused into the epilogue:
 * out = act([bias +] a @ bt^T), the activation evaluated on the fp32 accumulator
 * (after the bias) before the single rounding to the output type.  Generalises the
 * reference's one fused-sigmoid kernel (the 4096-cube sigmoid matmul its Inductor
 * scheduling fuses, ayla/torch_compile.py:532-547; math
 * ayla/passes/lower_to_ptx_template.py:84-113, :296-315) to every shape, op and schedule.
 * All other arguments as for ayla_b200_gemm.
 */
AYLA_B200_API int ayla_b200_gemm_act(int op, int dtype, int activation, const void* bias, const void* a,
                                     const void* bt, void* out, int64_t batch, int64_t m, int64_t n,
                                     int64_t k, const ayla_b200_config* cfg, void* workspace,
                                     size_t workspace_bytes, uint32_t* status, void* stream);

/*
 * ayla_b200_gemm_act with a gate: out = act([bias +] a @ bt^T) * mul, where `mul` has the shape,
 * type and layout of `out` (NULL = no gate) and enters in fp32 before the single rounding.  It
 * serves gated projections such as sigmoid(x @ Wg^T) * v, the producer half of the
 * `mm -> sigmoid -> mul -> mm` region the reference's Inductor pass recognises but has no kernel
 * for (ayla/torch_compile.py:288-504).  `mul` must not alias `out`.
 */
AYLA_B200_API int ayla_b200_gemm_act_mul(int op, int dtype, int activation, const void* bias, const void* a,
                                         const void* bt, const void* mul, void* out, int64_t batch, int64_t m,
                                         int64_t n, int64_t k, const ayla_b200_config* cfg, void* workspace,
                                         size_t workspace_bytes, uint32_t* status, void* stream);

/*
 * ayla_b200_gemm_act with one factor per output row: out[b][i][j] = act([bias +] a @ bt^T)[b][i][j]
 * * row_mul[b][i], where `row_mul` holds batch * m elements of the operands' type, contiguous,
 * and enters in fp32 before the single rounding.  With act = NONE and no bias this is a GEMM whose
 * left operand carries a per-row scale, e.g. the 1/rms factor of an RMSNorm whose weight vector has
 * been folded into `bt`: rmsnorm(x) @ W^T = rsqrt(mean(x^2) + eps)[i] * (x @ (W * g)^T).  The
 * reference lists epilogue fusion as an aim (README.md:6-7) and has no kernel of this form.
 */
AYLA_B200_API int ayla_b200_gemm_act_rowmul(int op, int dtype, int activation, const void* bias, const void* a,
                                            const void* bt, const void* row_mul, void* out, int64_t batch,
                                            int64_t m, int64_t n, int64_t k, const ayla_b200_config* cfg,
                                            void* workspace, size_t workspace_bytes, uint32_t* status,
                                            void* stream);

/*
 * Size of the scratch array built into the library for
 * ayla_b200_gemm_static_scratch: 8 MiB of device memory on every GPU that loads
 * the library, held until the process exits.
 */
#define AYLA_B200_STATIC_SCRATCH_BYTES (8u << 20)

/*
 * ayla_b200_gemm for callers that have no device memory to lend and may not
 * allocate any.  (No counterpart in the reference, which never needs scratch:
 * it has no split-K schedule.)
 *
 * Who needs it: a host that drives this library from inside another runtime's
 * memory regime -- an inference server or framework plugin that owns a fixed
 * pool and forbids cudaMalloc underneath it (cudaMalloc and cudaFree stall the
 * whole device and bypass the pool's accounting), or code that only ever sees the
 * operand pointers of one op and has nowhere to keep a workspace between calls.
 * For them the partial sums and arrival counters of a split-K schedule live in a
 * fixed array of AYLA_B200_STATIC_SCRATCH_BYTES inside the library image; the
 * caller passes operands and output only.  The call allocates nothing: no
 * cudaMalloc, no cudaFree, no allocating library routine.
 *
 * Same arguments and results as ayla_b200_gemm without the workspace pair.
 * A schedule whose scratch need exceeds the array is refused with
 * AYLA_B200_E_WORKSPACE and a message naming both sizes (schedules with
 * split_k == 1 need none and always fit).
 *
 * There is no activation, gate or SwiGLU form of this entry point: it covers
 * mm, addmm and bmm as ayla_b200_gemm does, nothing fused after them.
 *
 * The array's device address is resolved once per device (a runtime query made
 * with that device current): by ayla_b200_init, and again lazily by the first
 * call on a device that needs scratch should init not have done it; make that
 * first call outside stream capture.  All calls on a GPU share the one array and it keeps the previous
 * call's contents: the entry point clears the arrival counters on `stream`
 * before each launch, and two calls whose kernels can overlap on the GPU
 * (different streams, no dependency) race on it -- serialise them.
 */
AYLA_B200_API int ayla_b200_gemm_static_scratch(int op, int dtype, const void* bias, const void* a,
                                                const void* bt, void* out, int64_t batch, int64_t m,
                                                int64_t n, int64_t k, const ayla_b200_config* cfg,
                                                uint32_t* status, void* stream);

/*
 * out[M,N] = silu(x[M,K] @ w_gate[N,K]^T) * (x @ w_up[N,K]^T), both products kept
 * in fp32 until one final rounding.  One kernel, one pass over x; the
 * intermediates never reach HBM.  New op; its precedent is the reference's fused
 * matmul+sigmoid op (ayla/gemm_collection/auto_matmul_4096_wgmma256_wg_sigmoid.py:22-142)
 * and its silu/mul lowerings (ayla/passes/lower_to_ptx_template.py:296-315, :62-81).
 * Only cfg->cta_group, group_m, grid_ctas and the L2 hints are used.
 */
AYLA_B200_API int ayla_b200_swiglu(int dtype, const void* x, const void* w_gate, const void* w_up, void* out,
                     int64_t m, int64_t n, int64_t k, const ayla_b200_config* cfg, uint32_t* status,
                     void* stream);

/*
 * The schedule ayla_b200_gemm uses when cfg == NULL.  Counterpart of
 * select_gemm_schedule's fallback (ayla/gemm_jit.py:225-264).
 */
AYLA_B200_API int ayla_b200_default_config(int op, int dtype, int64_t batch, int64_t m, int64_t n, int64_t k,
                             ayla_b200_config* cfg_out);

/*
 * 0 if `cfg` can run the given problem, else an error code (message in
 * ayla_b200_last_error).  Counterpart of _legal (ayla/gemm_jit.py:115-138).
 */
AYLA_B200_API int ayla_b200_config_valid(const ayla_b200_config* cfg, int op, int dtype, int64_t batch, int64_t m,
                           int64_t n, int64_t k);

/* Bytes of workspace `cfg` needs for the problem (0 when split_k == 1). */
AYLA_B200_API size_t ayla_b200_workspace_bytes(const ayla_b200_config* cfg, int op, int64_t batch, int64_t m,
                                 int64_t n, int64_t k);

/*
 * Leading bytes of that workspace that must be zero before the first launch (the
 * split-K arrival counters; 64 KiB for every shape, so a workspace zeroed once can
 * be shared by launches of different shapes).  The kernel returns them to zero.
 */
AYLA_B200_API size_t ayla_b200_workspace_counter_bytes(const ayla_b200_config* cfg, int op, int64_t batch,
                                         int64_t m, int64_t n, int64_t k);

/*
 * Strided device-to-device copy on the copy engines (no SMs): `rows` rows of `width_bytes`,
 * source rows `src_pitch` apart, destination rows `dst_pitch` apart.  Used by the N-sharded
 * multi-GPU mm to put gathered column blocks of `out` in place while the GEMM of the next
 * row panel owns the SMs.  The reference is single-GPU and has no counterpart.
 */
AYLA_B200_API int ayla_b200_copy_2d(void* dst, size_t dst_pitch, const void* src, size_t src_pitch,
                                    size_t width_bytes, size_t rows, void* stream);

/*
 * Number of compiled kernel variants, and a description of variant i.  The listing covers the
 * variants without the activation epilogue; every one of them except the two SwiGLU kernels
 * exists a second time with it (used by ayla_b200_gemm_act).
 */
AYLA_B200_API int ayla_b200_kernel_count(void);
AYLA_B200_API int ayla_b200_kernel_info(int i, int32_t* tile_n, int32_t* cta_group, int32_t* epilogue,
                          int32_t* transposed_out, int32_t* stages, int32_t* smem_bytes);

/* Bound, in milliseconds, on every device-side wait (default 2000). */
AYLA_B200_API void ayla_b200_set_wait_timeout_ms(int64_t ms);

/*
 * Test hooks.  Bit 0: the TMA producers of every later launch issue no loads, so the MMA
 * warp's bounded wait for operands runs out (after the wait timeout) and the launch ends
 * normally with code 2 in `status` and garbage in `out`; the context stays usable.
 * Bit 1: cluster split-K launches keep all their ring slots and let the inbox of partial sums
 * overlay them (the form used when the ring could not spare the slots), so that both forms of
 * the exchange can be compared on one shape.  0 restores normal operation.
 */
AYLA_B200_API void ayla_b200_debug_set_flags(int flags);

/*
 * Launch overlap (on by default).  Every launch is issued with programmatic stream
 * serialisation: when the previous operation in the stream is also a kernel, the new grid's
 * CTAs may become resident and run their set-up (barrier initialisation, TMEM allocation,
 * descriptor fetch) while that kernel drains; the kernel then executes griddepcontrol.wait,
 * which returns only when the previous kernel has completed and its writes are visible,
 * before it touches global memory.  Results are the same as with plain stream order.
 * 0 switches to plain launches.  No counterpart in the reference (its launcher issues
 * plain cuLaunchKernel calls, ayla/ptx_runtime.py:237-282).
 */
AYLA_B200_API void ayla_b200_set_launch_overlap(int enabled);

AYLA_B200_API const char* ayla_b200_last_error(void);
AYLA_B200_API const char* ayla_b200_version(void);

#ifdef __cplusplus
}
#endif

#endif /* AYLA_B200_H_ */
