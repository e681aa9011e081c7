/*
 * tempest_b200.h -- C ABI of the B200 (sm_100a) kernel backend for Tempest.jl's
 * fused-kernel hot path.
 *
 * Every entry point takes raw device pointers (a CUdeviceptr from Julia's
 * `pointer(buffer)`), extents and strides in ELEMENTS, a dtype code and the
 * CUDA stream (a cudaStream_t passed as void*) of the calling task.  Unless
 * its comment says otherwise an entry point only enqueues work on that
 * stream: it does not allocate, synchronise or keep state between calls, so a
 * call can sit inside a stream capture (Tempest records its launches into a
 * CUDA graph, ext/CUDAExt.jl:515-545).  Every entry point returns TB200_OK or
 * a negative tb200_status; none of them aborts or traps.  A Tempest
 * `build_claim`/`build` turns a non-zero status into a throw, which makes the
 * cover fall to its next option (src/Compiler/cover/choose.jl:1014-1028).
 *
 * Layout convention: Julia arrays are dense column-major
 * (src/Compiler/IR/layout.jl:22-29).  A Julia (n, rows) matrix folded over its
 * first axis is passed as rows x n with the folded axis innermost; `ld` is the
 * distance between consecutive rows in elements (ld == n when dense).
 */
#ifndef TEMPEST_B200_H
#define TEMPEST_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum tb200_dtype {
    TB200_F32 = 0,
    TB200_BF16 = 1,
    TB200_F16 = 2    /* products only (ext/cuBLASExt.jl:64-65, test/cuda/products.jl:25-30) */
} tb200_dtype;

typedef enum tb200_status {
    TB200_OK = 0,
    TB200_ERR_NULL = -1,        /* a required pointer is null */
    TB200_ERR_SHAPE = -2,       /* an extent or stride is out of range */
    TB200_ERR_DTYPE = -3,       /* unknown or unsupported element type */
    TB200_ERR_ALIGN = -4,       /* a pointer is not aligned to its element type */
    TB200_ERR_WORKSPACE = -5,   /* workspace missing or too small */
    TB200_ERR_CUDA = -6,        /* a CUDA call failed; see tb200_last_cuda_error */
    TB200_ERR_UNSUPPORTED = -7, /* valid request the library has no kernel for */
    TB200_ERR_DEVICE = -8       /* the current device is not compute capability 10.x */
} tb200_status;

/* Library version (major*10000 + minor*100 + patch). No reference counterpart. */
int tb200_version(void);
/* Text of a tb200_status. No reference counterpart. */
const char *tb200_strerror(int status);
/* Text of the CUDA error behind the calling thread's last TB200_ERR_CUDA. */
const char *tb200_last_cuda_error(void);
/* Number of SMs of the current device (the grid-sizing unit). Replaces the
 * device query of ext/CUDAExt.jl:959 (RESIDENT_LANES per SM). */
int tb200_sm_count(void);

/* ---- fused row reductions (softmax, LayerNorm, forward and backward) -------
 * These replace the kernels ext/cuTileExt/build.jl:138-286 (`unsplit_kernel`,
 * resident and streamed sketches) and :560-705 (split + merge) generate for
 * the reduction groups of softmax_columns / layernorm and their derivatives
 * (test/fixtures/programs.jl:8, 13-17), and the floor kernels of
 * src/Compiler/codegen/scalar.jl:200-256.
 */

/* Operators of tb200_rowop_workspace_bytes. */
typedef enum tb200_rowop {
    TB200_SOFTMAX_FWD = 0,
    TB200_SOFTMAX_BWD = 1,
    TB200_LAYERNORM_FWD = 2,
    TB200_LAYERNORM_BWD = 3
} tb200_rowop;

/* Bytes of scratch the operator may need for rows x n elements of `dtype` on
 * the current device; 0 for most shapes (a row of up to 16384 elements is
 * folded in registers).  Non-zero for rows long enough to take the two-pass
 * split schedule and for the LayerNorm backward's dgamma/dbeta partial sums.
 * Replaces the partial-state workspace the reference sizes in
 * ext/cuTileExt/build.jl:560-609 (`split_kernels`).  A `build_claim` calls it
 * once and keeps the buffer alive with the launch (build.jl:957-961). */
size_t tb200_rowop_workspace_bytes(int rowop, int64_t n, int64_t rows, int dtype);

/* y[r, :] = exp(x[r, :] - lse_r), lse_r = logsumexp(x[r, :]).
 * lse (optional) receives lse_r in Float32 (stat_dtype TB200_F32) or in the
 * element type (TB200_BF16), the type the fold's value has in a Tempest plan
 * (src/Compiler/IR/folds.jl:42-55).  y may alias x (the row is read whole
 * before it is written: `in_place`, src/Compiler/Implement/Implement.jl:195-202)
 * unless the shape takes the split schedule.  An empty row gives lse = -Inf
 * (folds.jl:184).  workspace: tb200_rowop_workspace_bytes bytes, 16-byte
 * aligned, or NULL when that is 0. */
int tb200_softmax_fwd(const void *x, void *y, void *lse, int64_t n, int64_t rows, int64_t ld,
                      int dtype, int stat_dtype, void *workspace, size_t workspace_bytes,
                      void *stream);

/* dx = y * (dy - sum(y * dy)) per row.  With lse == NULL `y_or_x` holds the
 * forward's output y; otherwise it holds x and y = exp(x - lse) is recomputed
 * (the planner's save-or-recompute choice, src/Compiler/plan/partition.jl).
 * dx may alias dy or y_or_x under the resident schedule. */
int tb200_softmax_bwd(const void *y_or_x, const void *lse, const void *dy, void *dx, int64_t n,
                      int64_t rows, int64_t ld, int dtype, int stat_dtype, void *workspace,
                      size_t workspace_bytes, void *stream);

/* y = (x - mean) * rstd * gamma (+ beta); mean and variance of each row from
 * one read of it (the reference's Relative{Square} fold,
 * src/Compiler/IR/folds.jl:143, 166-182).  beta, mean, rstd may be NULL; mean
 * and rstd are Float32 [rows]; gamma and beta have the element type. */
int tb200_layernorm_fwd(const void *x, const void *gamma, const void *beta, void *y, float *mean,
                        float *rstd, float eps, int64_t n, int64_t rows, int64_t ld, int dtype,
                        void *workspace, size_t workspace_bytes, void *stream);

/* dx = rstd * (gh - mean(gh) - xh * mean(gh * xh)), gh = dy * gamma,
 * xh = (x - mean) * rstd; dgamma[i] = sum over rows of dy * xh and
 * dbeta[i] = sum over rows of dy, in the element type: per-block partial sums
 * in the workspace merged by a second launch in a fixed order (the
 * reference's partial folds and merge kernel, ext/cuTileExt/emit.jl:744-753,
 * build.jl:654-696), so results repeat bit for bit.
 * mean/rstd NULL: recomputed from x.  dgamma and dbeta both NULL: no workspace
 * is needed for rows the resident schedule holds (up to 8192 elements with
 * 128-bit accesses, 4096 without).  Longer rows are streamed: one block walks
 * a row three or four times through L2, a second kernel takes the column sums
 * over row slabs; that form keeps recomputed statistics and the slabs'
 * partial sums in the workspace (tb200_rowop_workspace_bytes covers it). */
int tb200_layernorm_bwd(const void *x, const void *gamma, const void *dy, const float *mean,
                        const float *rstd, void *dx, void *dgamma, void *dbeta, float eps,
                        int64_t n, int64_t rows, int64_t ld, int dtype, void *workspace,
                        size_t workspace_bytes, void *stream);

/* tb200_layernorm_bwd without a workspace argument, for callers that cannot
 * supply scratch memory: programs whose device buffers were all laid out
 * before the kernels were chosen and that have no allocator to turn to at call
 * time, or that must stay clear of the driver's allocator (it takes a
 * process-wide lock and may wait for the device).  The partial dgamma/dbeta
 * sums go to an 8 MiB array built into the library, which every GPU that loads
 * the library keeps resident until the process ends.  Rows longer than
 * tb200_layernorm_bwd_noalloc_max_row() elements (8192) are refused with
 * TB200_ERR_WORKSPACE, and so are rows of more than 4096 elements that cannot
 * be read with 128-bit accesses (x, gamma, dy or dx not 16-byte aligned, or n
 * or ld not a multiple of 4 Float32 / 8 BFloat16 elements): such rows do not fit
 * one block's registers.  The entry point itself allocates nothing.
 * The first call on each device looks up the array's device address; make that
 * call outside any stream capture.  Every call on a device uses the same
 * array: calls whose kernels could overlap on the GPU (two streams) corrupt
 * each other's sums, so the caller must order them.  Results equal
 * tb200_layernorm_bwd's dx exactly and its dgamma/dbeta up to the order of
 * the partial sums.  This entry point has no counterpart in the reference. */
size_t tb200_layernorm_bwd_noalloc_max_row(void);
int tb200_layernorm_bwd_noalloc(const void *x, const void *gamma, const void *dy, const float *mean,
                                const float *rstd, void *dx, void *dgamma, void *dbeta, float eps,
                                int64_t n, int64_t rows, int64_t ld, int dtype, void *stream);

/* ---- products with fused epilogues ----------------------------------------
 * C = epilogue(alpha * A * B), row-major C[M][N].  Replaces the generated
 * `:product` kernels of ext/cuTileExt/contract.jl:112-161 with their fused
 * outputs (ext/cuTileExt/build.jl:243-246) and the library calls of
 * ext/cuBLASExt.jl:247-259 (`cublasGemmStridedBatchedEx`), including its
 * `accumulated` template D .+ A*B (cuBLASExt.jl:25-29).
 *
 * Operand layouts cover cuBLAS's four transposes (cuBLASExt.jl:70-80): an
 * operand is K-major when its contracted axis is contiguous (A stored [M][K],
 * B stored [N][K]) and MN-major otherwise (A stored [K][M], B stored [K][N]).
 * A Julia `w::(out,in)` is memory [in][out]: for y = w*x it is an MN-major B.
 */
typedef enum tb200_layout {
    TB200_K_MAJOR = 0,
    TB200_MN_MAJOR = 1
} tb200_layout;

typedef enum tb200_epilogue {
    TB200_EPI_NONE = 0,          /* alpha * acc */
    TB200_EPI_BIAS = 1,          /* alpha * acc + bias[n] */
    TB200_EPI_BIAS_GELU = 2,     /* gelu_tanh(alpha * acc + bias[n]); aux_out <- the value before gelu */
    TB200_EPI_BIAS_TANH = 3,     /* tanh(alpha * acc + bias[n]) */
    TB200_EPI_MUL_GELU_GRAD = 4, /* alpha * acc * gelu_tanh'(aux[m][n]): the pullback through the activation */
    TB200_EPI_MUL_TANH_GRAD = 5, /* alpha * acc * (1 - aux[m][n]^2), aux = tanh's output */
    TB200_EPI_AXPY = 6           /* aux[m][n] + alpha * acc (aux in the output type; may alias C) */
} tb200_epilogue;

typedef struct tb200_gemm_desc {
    int64_t m, n, k;
    int64_t lda, ldb, ldc;       /* leading dimensions in elements */
    int64_t ld_aux, ld_aux_out;
    int a_layout, b_layout;      /* tb200_layout */
    int in_dtype, out_dtype;     /* tb200_dtype; bias and aux have in_dtype (aux of AXPY: out_dtype) */
    int epilogue;                /* tb200_epilogue */
    float alpha;
    int tile_n;                  /* 0 = choose; 128 or 256 = the variant the tuner picked
                                    (the counterpart of TEMPEST_PRODUCT_TILE, ext/cuTileExt/contract.jl:36-49);
                                    512 = tiles of 256 x 256 computed by pairs of CTAs on neighbouring SMs
                                    (each loads half of either operand's tile); -1 = choose among the single-CTA
                                    tiles only */
    int force_simt;              /* 1 = the generic kernel (Float32-exact, any alignment) */
    int direct_epilogue;         /* 1 = each thread stores its own output row instead of staging
                                    tiles in shared memory and writing whole lines (a tuner variant) */
    /* A batch of alike products in one launch, as cublasGemmStridedBatchedEx takes them
     * (ext/cuBLASExt.jl:247-259): member i reads a + i * stride_a, b + i * stride_b and writes
     * c + i * stride_c (elements).  batch 0 or 1 = one product.  A zero stride of an operand that is
     * only read shares it among the members (one weight matrix for every member). */
    int64_t batch;
    int64_t stride_a, stride_b, stride_c;
    int64_t stride_bias, stride_aux, stride_aux_out;
    /* Split-K: the sum over k cut into `split_k` ranges whose Float32 partial results are merged in
     * range order by a second launch (ext/cuTileExt/contract.jl:89-94, `product_split`; the merge is
     * ext/cuTileExt/build.jl:654-696).  0 = the library decides (it splits when the output has too
     * few tiles to fill a quarter of the SMs and k is long), 1 = never, s > 1 = s ranges at most.
     * A split needs `workspace` (tb200_gemm_workspace_bytes, 16-byte aligned); without one the
     * product runs unsplit. */
    int split_k;
    void *workspace;
    size_t workspace_bytes;
    /* Test hook, 0 in production.  Bit 0: the loading thread of the tensor-core kernel withholds its
     * tiles and every bounded wait gives up after 20 ms instead of 2 s, so that the failure path (an
     * error code in tb200_device_error, the launch returning, the context still usable) can be
     * exercised without a fault. */
    int debug;
} tb200_gemm_desc;

/* Products alike by arrays of their operands' addresses: `count` products of the descriptor's shape, layouts and
 * element types, member i reading a[i], b[i] and writing c[i]; a, b, c are DEVICE arrays of `count` device addresses
 * (the reference's `Products`, ext/cuBLASExt.jl:273-306: cublasGemmBatchedEx on arrays it rewrites in `repoint!`).
 * Plain products only (epilogue NONE, C = alpha * A * B with alpha 0 read as 1); the descriptor's batch, split and
 * workspace fields are ignored.  BFloat16 or Float16 operands run as warp-level MMAs, any alignment and any
 * extents; Float32 operands (or force_simt) on the CUDA cores in Float32.  No workspace. */
int tb200_gemm_pointers(const tb200_gemm_desc *desc, const void *const *a, const void *const *b, void *const *c,
                        int64_t count, void *stream);

/* Bytes of scratch a split of this product wants (0 when it would not split). */
size_t tb200_gemm_workspace_bytes(const tb200_gemm_desc *desc);

/* The tile form the tensor-core path takes for a descriptor: 128 or 256 (columns of
 * a single CTA's 128-row tile) or 512 (256 x 256 tiles by pairs of CTAs), 0 for an
 * empty product.  Host arithmetic only; what sends a product to the CUDA-core
 * kernel instead (types, alignments) is not looked at. */
int tb200_gemm_tile_form(const tb200_gemm_desc *desc);

/* Enqueues the product.  BFloat16 or Float16 operands with 16-byte aligned bases and
 * leading dimensions (and batch strides) that are multiples of 8 run on the tensor cores
 * (tcgen05, Float32 accumulation, one rounding at the store); everything else
 * runs the generic kernel.  The tensor-core path builds its TMA descriptors
 * from the raw pointers on every call and passes them as kernel parameters;
 * tb200_gemm_plan_create below builds them once.  Float16 takes the epilogues
 * NONE, BIAS and AXPY on the tensor cores. */
int tb200_gemm(const tb200_gemm_desc *desc, const void *a, const void *b, void *c, const void *bias,
               const void *aux, void *aux_out, void *stream);

/* A prepared product: everything tb200_gemm works out per call (validation, schedule, the TMA
 * descriptors) done once, so that a launch is one kernel launch -- the C side of the reference's
 * `build` -> `launch()` / `repoint!` split (ext/cuBLASExt.jl:247-268, ext/cuTileExt/build.jl:949-976).
 * tb200_gemm_plan_repoint replaces one operand's address (tb200_gemm_operand) and rebuilds what
 * depends on it; the new address must be aligned as the old one was (src/Compiler/Implement/
 * Implement.jl:162-175).  A plan belongs to the device that was current when it was created, may be
 * launched any number of times on any stream of that device, and is not to be repointed while
 * another thread launches it.  Creating a plan allocates eight bytes of device memory (launching
 * allocates nothing): two counters from which the persistent blocks draw their tiles, so that a block
 * which reaches its SM late -- a communication kernel was running there -- takes fewer tiles instead of
 * holding the launch up; because of them two launches of ONE plan must not overlap on the GPU (launch
 * a plan on one stream at a time, or create two plans). */
typedef struct tb200_gemm_plan tb200_gemm_plan;
typedef enum tb200_gemm_operand {
    TB200_GEMM_A = 0, TB200_GEMM_B = 1, TB200_GEMM_C = 2, TB200_GEMM_BIAS = 3, TB200_GEMM_AUX = 4,
    TB200_GEMM_AUX_OUT = 5, TB200_GEMM_WORKSPACE = 6
} tb200_gemm_operand;
int tb200_gemm_plan_create(const tb200_gemm_desc *desc, const void *a, const void *b, void *c, const void *bias,
                           const void *aux, void *aux_out, tb200_gemm_plan **plan);
int tb200_gemm_plan_launch(const tb200_gemm_plan *plan, void *stream);
int tb200_gemm_plan_repoint(tb200_gemm_plan *plan, int operand, const void *address);
void tb200_gemm_plan_destroy(tb200_gemm_plan *plan);

/* Measures the compiled-in tile variants of one product on its own operands
 * and returns the faster tile_n (128, 256 or 512) to put in the descriptor, or a
 * negative status: the measured stage of the reference's search over a claim's
 * variants (src/Compiler/Implement/Implement.jl:120,
 * ext/cuTileExt/contract.jl:171-235) over what this library holds.  Overwrites C
 * (and aux_out) with the product's own result, synchronises the stream; call it
 * while building, not inside a capture. */
int tb200_gemm_tune(const tb200_gemm_desc *desc, const void *a, const void *b, void *c, const void *bias,
                    const void *aux, void *aux_out, void *stream);

/* The wider search: times every compiled-in variant of the product -- tile widths 128 / 256, the
 * sum unsplit or split (when a workspace is given), results stored through shared memory and TMA or
 * by each thread -- and writes the fastest one's tile_n, split_k and direct_epilogue into *desc.
 * Same rules as tb200_gemm_tune (overwrites C, synchronises, not for a capture).  Returns
 * TB200_OK or a negative status. */
int tb200_gemm_tune_desc(tb200_gemm_desc *desc, const void *a, const void *b, void *c, const void *bias,
                         const void *aux, void *aux_out, void *stream);

/* Synchronises the device, then returns and clears the code a tensor-core
 * product kernel recorded if one of its bounded waits gave up (0 = none).  No
 * reference counterpart: Tempest's kernels have no device-side waits. */
int tb200_device_error(void);

/* ---- attention -----------------------------------------------------------------
 * Arrays are the reference's (features, heads, positions, batch) Julia arrays
 * (test/fixtures/operations.jl:21-29), i.e. dense memory
 * [batch][position][head][feature]; the log-sum-exp is (1, heads, queries, batch),
 * memory [batch][query][head], Float32.  Query head h reads key/value head
 * h / (heads / kv_heads). */
typedef struct tb200_attn_desc {
    int batch, heads, kv_heads;
    int queries, keys, head_dim;
    int causal;                  /* keys after a query masked out (key index <= query index kept) */
    float scale;                 /* scores are scale * q.k ; 1/sqrt(head_dim) in the reference */
    int dtype;                   /* TB200_BF16 */
    int deterministic;           /* the pullback only: 0 = one kernel whose dq contributions are added into a
                                    Float32 workspace in whatever order the key tiles finish (the reference's
                                    default, `CUDATarget(...; deterministic = false)`,
                                    src/Compiler/runtime/target.jl:31); 1 = two kernels, no atomic adds, results
                                    repeat bit for bit */
    int value_dim;               /* features of v, o, dout and dv when they differ from head_dim (the queries' and
                                    keys'), as multi-head latent attention's do (test/cuda/attention.jl:150-177;
                                    `own_domain`, src/Compiler/Implement/groups.jl:211-219); 0 = head_dim.  Such
                                    programs run the CUDA-core kernels (dense arrays, both up to 256 features) */
} tb200_attn_desc;

/* o = softmax(scale * k'q + mask) weighted sum of v, lse beside it (NULL: not
 * stored).  Scores and softmax in Float32 from the BFloat16 queries and keys,
 * weights rounded to BFloat16 for the second product, output rounded once: what
 * the reference's generated kernel (ext/cuTileExt/build.jl:419-488,
 * ext/cuTileExt/emit.jl:1079-1135) and its cuDNN call (ext/cuDNNExt.jl:116-132,
 * 186-210) compute.  head_dim 128 on the tensor-core path; other sizes:
 * TB200_ERR_UNSUPPORTED. */
int tb200_attention_fwd(const tb200_attn_desc *desc, const void *q, const void *k, const void *v,
                        void *o, float *lse, void *stream);

/* As tb200_device_error, for the attention kernels. */
int tb200_attention_device_error(void);

size_t tb200_attention_bwd_workspace_bytes(const tb200_attn_desc *desc);

/* The pullback of tb200_attention_fwd for upstream dout: dq, dk, dv (BFloat16,
 * laid out as q, k, v).  Recomputes the scores, P = exp(s - lse), with
 * delta = sum_d dout*o from the output as stored (the reference's
 * `rounded_backward`, docs/src/cuda.md:54-63); P and dS enter their products
 * rounded to BFloat16 (docs/src/cuda.md:40-46).  Two forms, chosen by
 * desc->deterministic as the reference's `CUDATarget(...; deterministic)` chooses
 * (src/Compiler/runtime/target.jl:31):
 *   0  one kernel per key tile over the queries that keeps dk and dv in tensor
 *      memory and adds each step's dq contribution into a Float32 accumulator in
 *      the workspace, then a kernel that rounds it (ext/cuTileExt/transpose.jl:
 *      165-187 `added_folds` / `add_step!`, :201-213 `late_kernel`): five products
 *      per step; dq repeats to Float32 rounding, not bit for bit;
 *   1  dk and dv folded per key tile over the queries, dq by a second kernel per
 *      query tile over the keys, no atomic adds, results repeat bit for bit
 *      (ext/cuTileExt/build.jl:295-318): seven products.
 * workspace: tb200_attention_bwd_workspace_bytes bytes (it depends on the form),
 * 16-byte aligned.  Head dimensions other than 128 run the CUDA-core kernels,
 * which are deterministic either way. */
int tb200_attention_bwd(const tb200_attn_desc *desc, const void *q, const void *k, const void *v,
                        const void *o, const float *lse, const void *dout, void *dq, void *dk,
                        void *dv, void *workspace, size_t workspace_bytes, void *stream);

/* Which kernels a descriptor is computed by -- host arithmetic only, nothing is
 * launched and no device is needed: what `claims` can say about a group before it is
 * built.  `masked`: the call carries masks the device holds (tb200_attn_mask with
 * starts or lengths); `pullback`: the gradient entry rather than the forward.
 * Returns a TB200_ATTN_FORM_* value, or the negative status the entry itself would
 * return for the descriptor (pointer alignment, which the entries also look at, is
 * the caller's: Tempest's buffers are 128-byte aligned). */
#define TB200_ATTN_FORM_CUDA_CORES 0   /* a warp per query (or key), Float32, any geometry up to 256 features */
#define TB200_ATTN_FORM_TILE 1         /* tensor cores, one 128-query tile per block (forward) */
#define TB200_ATTN_FORM_TWO_TILES 2    /* tensor cores, two query tiles per block (forward, more than one tile, no device-held mask) */
#define TB200_ATTN_FORM_ONE_KERNEL 3   /* pullback on the tensor cores, dQ added by TMA reductions (deterministic = 0) */
#define TB200_ATTN_FORM_TWO_KERNELS 4  /* pullback on the tensor cores, dK/dV and dQ kernels (deterministic = 1) */
int tb200_attention_form(const tb200_attn_desc *desc, int masked, int pullback);

/* Times both forms on these operands and returns the `deterministic` value (0 or 1)
 * of the faster one, or a negative status: the measured stage of the reference's
 * search over a claim's variants (src/Compiler/Implement/Implement.jl:120) over the
 * library's two schedules.  For callers that accept either form.  Overwrites dq, dk,
 * dv with the pullback's result, synchronises the stream (call it while building,
 * not inside a capture); workspace sized for deterministic = 0. */
int tb200_attention_bwd_tune(const tb200_attn_desc *desc, const void *q, const void *k, const void *v,
                             const void *o, const float *lse, const void *dout, void *dq, void *dk,
                             void *dv, void *workspace, size_t workspace_bytes, void *stream);

int tb200_attention_bwd_device_error(void);

/* As tb200_device_error, for the DeltaNet scans, whose tiles arrive by TMA on an mbarrier: 0, or 1 (forward scan) /
 * 2 (reverse scan) when a wait gave up. */
int tb200_deltanet_device_error(void);

/* As tb200_device_error, for the row kernels that wait on bulk copies into shared memory (the LayerNorm
 * backward of 1024-, 2048- and 4096-long rows with saved statistics): 0, or 1 when a wait gave up. */
int tb200_rows_device_error(void);

/* All the error words in one call: synchronises the device, returns
 * product | attention forward << 8 | attention backward << 16 | row kernels << 24 | DeltaNet scans << 28 (0 = every bounded
 * wait completed) and clears them, or a negative status.  The launch entry
 * points return TB200_OK once their kernels are enqueued, so a wait that gives
 * up later is visible only here: a caller polls this wherever it synchronises
 * anyway (after a step, before it reads results back) and treats a non-zero
 * value as a failed launch whose outputs must not be used.  No reference
 * counterpart. */
int tb200_device_errors(void);

/* Masks the device holds, and operands at other strides.  Two of the reference's
 * mask programs (test/cuda/attention.jl:217-246, 248-275; the scheduling side is
 * ext/cuTileExt/mask.jl:299-353):
 *   packed documents -- with `causal`, query j sees keys doc_start[b][j] <= i <= j
 *     (0-based here; FlashAttention's variable-length batches);
 *   lengths -- keys at and beyond kv_len[b] are masked (decode over a cache).
 * A query that sees no key gets a zero output and a log-sum-exp of -Inf.
 * Strides are in elements over (batch, position, head) with the features
 * contiguous; all zero = the dense [batch][position][head][feature] default.  A
 * key cache laid out (features, positions, key heads, sequences) is
 * kv_stride = {kv_heads * keys * d, d, keys * d}.  The forward with 128 features
 * runs on the tensor cores (strides that are multiples of 8 elements, 16-byte
 * aligned arrays): every query tile finds the key tiles it has to visit from its
 * queries' starts and the sequence's length, and masks the tiles those fall in
 * row by row.  Other head dimensions (up to 256), other strides and the pullback
 * run the CUDA-core kernels. */
typedef struct tb200_attn_mask {
    const int32_t *doc_start;   /* [batch][queries] or NULL */
    const int32_t *kv_len;      /* [batch] or NULL */
    int64_t q_stride[3];        /* q, o, dq, dout */
    int64_t kv_stride[3];       /* k, v, dk, dv */
} tb200_attn_mask;

int tb200_attention_fwd_masked(const tb200_attn_desc *desc, const tb200_attn_mask *mask, const void *q,
                               const void *k, const void *v, void *o, float *lse, void *stream);
int tb200_attention_bwd_masked(const tb200_attn_desc *desc, const tb200_attn_mask *mask, const void *q,
                               const void *k, const void *v, const void *o, const float *lse, const void *dout,
                               void *dq, void *dk, void *dv, void *stream);

/* The masked pullback on the tensor cores: 128 features, dense arrays (a mask
 * with strides, another head dimension: TB200_ERR_UNSUPPORTED, for which the
 * entry above remains), in either of the pullback's forms (desc->deterministic).
 * Keys beyond a sequence's length and key tiles that lie wholly beyond it are
 * skipped; with packed documents a key tile stops at the last chunk of queries
 * that can see it and a query tile starts at the first keys any of its queries
 * sees (found from the smallest start of every 64 queries, so starts need not be
 * sorted), and steps in between take the element-by-element test only where a
 * start can hide a key.  The workspace is tb200_attention_bwd's plus a row of
 * starts per (batch, head) and their block minima and maxima. */
size_t tb200_attention_bwd_masked_workspace_bytes(const tb200_attn_desc *desc);
int tb200_attention_bwd_masked_ws(const tb200_attn_desc *desc, const tb200_attn_mask *mask, const void *q,
                                  const void *k, const void *v, const void *o, const float *lse, const void *dout,
                                  void *dq, void *dk, void *dv, void *workspace, size_t workspace_bytes,
                                  void *stream);

/* ---- chunked gated DeltaNet ------------------------------------------------------
 * The program of examples/deltanet.jl:56-85: q, k (dk, T, heads) = memory
 * [head][t][dk], v (dv, T, heads), a (log decay) and beta (T, heads) in
 * Float32, result (T, dv, heads) = memory [head][dv][t].  Replaces the batched
 * products and the `:recurrence` kernel Tempest plans for it
 * (ext/cuTileExt/build.jl:772-835, ext/cuTileExt/cuTileExt.jl:831-852). */
typedef struct tb200_deltanet_desc {
    int heads;        /* batch * heads sequences */
    int positions;    /* T, a multiple of chunk */
    int dk, dv;       /* 128, 128 */
    int chunk;        /* 64 */
    int dtype;        /* TB200_BF16 for q, k, v and the result */
} tb200_deltanet_desc;

size_t tb200_deltanet_workspace_bytes(const tb200_deltanet_desc *desc);

/* Forward pass.  Other geometries than dk = dv = 128, chunk = 64: TB200_ERR_UNSUPPORTED. */
int tb200_deltanet_fwd(const tb200_deltanet_desc *desc, const void *q, const void *k, const void *v,
                       const float *a, const float *beta, void *o, void *workspace,
                       size_t workspace_bytes, void *stream);

size_t tb200_deltanet_bwd_workspace_bytes(const tb200_deltanet_desc *desc);

/* Pullback of the forward pass: given dout (the result's layout, [head][dv][t]
 * BFloat16) writes dq, dk [head][t][dk] and dv [head][t][dv] in BFloat16 and da,
 * dbeta [head][t] in Float32.  It runs the forward again inside (keeping the
 * state at every chunk start), so it needs no saved tensors, and stands for the
 * gradient program Tempest derives from the same source
 * (examples/deltanet.jl:96-101, src/Compiler/Differentiate).  Same geometry
 * limits as the forward. */
int tb200_deltanet_bwd(const tb200_deltanet_desc *desc, const void *q, const void *k, const void *v,
                       const float *a, const float *beta, const void *dout, void *dq, void *dk, void *dv,
                       float *da, float *dbeta, void *workspace, size_t workspace_bytes, void *stream);

/* ---- generic fused map -> fold groups ---------------------------------------
 * Any group of the kinds the four named row entries are instances of: a DAG of
 * scalar terms over a (n, rows) domain whose first, contiguous axis is folded,
 * with the folds' finished values readable by later terms.  It is the view the
 * reference hands every backend (`GroupView`, src/Compiler/Implement/groups.jl:
 * 106-125) cut down to row groups: terms follow src/Compiler/IR/terms.jl:12-87
 * (Load, Lit, Ix, Apply, Stat, Cast), folds follow src/Compiler/IR/folds.jl:
 * 66-89 (sum, max, min, prod), :123-198 (`Relative{Exponential}` = log-sum-exp,
 * `Relative{Square}` = mean and centred sum of squares by Welford/Chan).
 * Execution follows the reference's floor (src/Compiler/codegen/scalar.jl:
 * 200-256): per row, phase by phase, every fold of a phase in one sweep, then a
 * last sweep for the full-shape outputs -- here with the sweeps of one row
 * spread over a group of threads, re-reading the row from L1/L2, and the term
 * DAG run by a small interpreter in registers/local memory (Float32). */
enum { TB200_GROUP_MAX_INPUTS = 8, TB200_GROUP_MAX_TERMS = 48, TB200_GROUP_MAX_FOLDS = 8, TB200_GROUP_MAX_OUTPUTS = 8 };

typedef enum tb200_term_op {
    TB200_T_LOAD = 0,    /* a = input index */
    TB200_T_LIT = 1,     /* imm */
    TB200_T_INDEX = 2,   /* position along the folded axis, 0-based, as Float32 (Ix) */
    TB200_T_STAT = 3,    /* a = fold index of an earlier phase: its observed value for this row */
    TB200_T_STAT2 = 4,   /* the second observed value of TB200_FOLD_MEANVAR (the variance) */
    TB200_T_ADD = 5, TB200_T_SUB = 6, TB200_T_MUL = 7, TB200_T_DIV = 8, TB200_T_MAX = 9, TB200_T_MIN = 10,
    TB200_T_NEG = 11, TB200_T_EXP = 12, TB200_T_LOG = 13, TB200_T_TANH = 14, TB200_T_SQRT = 15,
    TB200_T_RSQRT = 16, TB200_T_ABS = 17, TB200_T_ABS2 = 18, TB200_T_RECIP = 19, TB200_T_SIGMOID = 20,
    TB200_T_FMA = 21,    /* a * b + c, fused */
    TB200_T_SELECT = 22, /* a > 0 ? b : c */
    TB200_T_ROUND_BF16 = 23, /* Cast to BFloat16 and back: the rounding an Apply of that eltype makes */
    /* The two below describe groups that tb200_group_route recognises and hands to a kernel of their own; the term
     * interpreter and the generator decline them. */
    TB200_T_RECOMPUTED = 24, /* sum over e < c of X[row][e] * Y[i][e]: a fold formed where it is read (Recomputed,
                                src/Compiler/IR/terms.jl:69-87) over one extra axis of extent c; a = input X of
                                shape TB200_SHAPE_ROW_VECTORS, b = input Y of shape TB200_SHAPE_ALONG_VECTORS */
    TB200_T_ROW_INDEX = 25,  /* the row's own position, 0-based, as Float32: with TB200_T_INDEX under a
                                TB200_T_SELECT it spells a mask on two positions (ext/cuTileExt/mask.jl:54-75) */
    TB200_T_STATE = 26       /* a = state index: the state's value before this step (recurrences only) */
} tb200_term_op;

typedef struct tb200_term { int op, a, b, c; float imm; } tb200_term;

typedef enum tb200_fold_kind {
    TB200_FOLD_SUM = 0, TB200_FOLD_MAX = 1, TB200_FOLD_MIN = 2, TB200_FOLD_PROD = 3,
    TB200_FOLD_LOGSUMEXP = 4, /* observes log(sum(exp(y))) from the online (max, rebased sum) state */
    TB200_FOLD_MEANVAR = 5,   /* observes the mean; TB200_T_STAT2 reads sum((y - mean)^2) / n */
    TB200_FOLD_WEIGHTED = 6   /* sum over i of term(i) * V[i][:], one vector per row: `payload` = input V of shape
                                 TB200_SHAPE_ALONG_VECTORS (the pair element of the attention fold; routed only) */
} tb200_fold_kind;

typedef struct tb200_fold { int kind, term, phase, payload; } tb200_fold;

typedef enum tb200_group_shape {
    TB200_SHAPE_FULL = 0,    /* (n, rows): element (i, row) at row * ld + i */
    TB200_SHAPE_ALONG = 1,   /* (n,): one value per position, shared by all rows (a LayerNorm weight) */
    TB200_SHAPE_PER_ROW = 2, /* (rows,): one value per row (a saved statistic) */
    TB200_SHAPE_SCALAR = 3,
    TB200_SHAPE_ROW_VECTORS = 4,   /* (ld, rows): a vector of ld elements per row (routed groups only) */
    TB200_SHAPE_ALONG_VECTORS = 5  /* (ld, n): a vector of ld elements per position along the row */
} tb200_group_shape;

typedef struct tb200_group_input { int shape, dtype; int64_t ld; } tb200_group_input;

/* from = 0: the term `index`, full shape, rounded once to `dtype`; from = 1 / 2: the
 * first / second observed value of fold `index`, one per row */
typedef struct tb200_group_output { int from, index, dtype; int64_t ld; } tb200_group_output;

typedef struct tb200_group_desc {
    int64_t n, rows;
    int n_inputs, n_terms, n_folds, n_outputs;
    tb200_group_input inputs[TB200_GROUP_MAX_INPUTS];
    tb200_term terms[TB200_GROUP_MAX_TERMS];     /* topologically ordered: arguments come before uses */
    tb200_fold folds[TB200_GROUP_MAX_FOLDS];     /* phase p may read TB200_T_STAT of phases < p */
    tb200_group_output outputs[TB200_GROUP_MAX_OUTPUTS];
} tb200_group_desc;

/* Checks a descriptor without running it: TB200_OK or the status the launch would return. */
int tb200_rowreduce_generic_check(const tb200_group_desc *desc);

/* inputs[i], outputs[j]: device addresses in the descriptor's order.  No workspace. */
int tb200_rowreduce_generic(const tb200_group_desc *desc, const void *const *inputs, void *const *outputs,
                            void *stream);

/* Groups with a kernel of their own.  tb200_group_route looks at the structure of a descriptor's terms, as the
 * reference's generator decides which of its sketches claims a group (ext/cuTileExt/cuTileExt.jl:899-929), and
 * answers which dedicated kernel computes it: the attention group of the reference's plans -- scores recomputed
 * over the features, optionally masked to the positions up to the row's own, their log-sum-exp, and the weights'
 * sum of the value rows (test/fixtures/operations.jl:21-76 as the planner groups it) -- is the one it knows.
 * tb200_group_attention runs such a descriptor: it states the computation at one (head, batch) of the domain's
 * outer axes (n = keys, rows = queries), `heads`, `kv_heads`, `batch` give those axes, and the inputs are the
 * reference's whole (features, heads, positions, batch) arrays; outputs as tb200_attention_fwd writes them. */
typedef enum tb200_route { TB200_ROUTE_NONE = 0, TB200_ROUTE_ATTENTION = 1, TB200_ROUTE_ATTENTION_CAUSAL = 2 } tb200_route;
int tb200_group_route(const tb200_group_desc *desc);
int tb200_group_attention(const tb200_group_desc *desc, int heads, int kv_heads, int batch, const void *const *inputs,
                          void *const *outputs, void *stream);

/* The same groups compiled: the descriptor is turned into CUDA source with its
 * extents, element types, alignment and schedule as constants, compiled for
 * sm_100a by NVRTC (loaded with dlopen on first use) and cached by descriptor --
 * the counterpart of the kernel the reference's generator emits and caches per
 * group (ext/cuTileExt/build.jl:138-286, ext/cuTileExt/cache.jl:59).  Rows that
 * fit in registers are read once and stay resident through every phase.
 * TB200_ERR_UNSUPPORTED when NVRTC cannot be loaded or the source does not
 * compile (tb200_rowreduce_compile_log holds the compiler's words); the
 * interpreter above then remains.
 *
 * tb200_rowreduce_compile compiles ahead of time and needs no device: bit i of
 * vector_inputs / vector_outputs promises that input / output i is aligned for
 * 128-bit accesses (base address and row pitch).  tb200_rowreduce_compiled works
 * those bits out from the addresses it is given, compiles on first use (so a
 * first call belongs outside a stream capture) and launches. */
int tb200_rowreduce_compile(const tb200_group_desc *desc, unsigned vector_inputs, unsigned vector_outputs);
int tb200_rowreduce_compiled(const tb200_group_desc *desc, const void *const *inputs, void *const *outputs,
                             void *stream);
/* The generated source (for inspection): returns the bytes needed including the
 * terminator, 0 for a descriptor that is refused; fills `buffer` when given. */
size_t tb200_rowreduce_source(const tb200_group_desc *desc, unsigned vector_inputs, unsigned vector_outputs,
                              char *buffer, size_t buffer_bytes);
const char *tb200_rowreduce_compile_log(void);

/* The same descriptors with every fold running over the rows -- the other, strided axis --
 * instead of along them: the bias gradient, LayerNorm's weight gradients, any sum over the
 * batch the planner forms.  The reference realises these as partial folds per block and a
 * merge kernel (ext/cuTileExt/emit.jl:729-753, ext/cuTileExt/build.jl:654-696); here one
 * generated kernel lets each thread own a column and fold the rows of its slab in order,
 * and a second merges the slabs in a fixed order, so results repeat bit for bit.  Terms are
 * evaluated per element as above (full, along, per-row and scalar inputs, the element's
 * index along the row) but may not read row statistics; folds: sum, max, min, prod; every
 * output is the value of one fold (from = 1), `n` elements of its dtype, rounded once.
 * workspace: tb200_colreduce_workspace_bytes bytes, 16-byte aligned.  Compiled by NVRTC on
 * first use and cached, as above (TB200_ERR_UNSUPPORTED without NVRTC). */
size_t tb200_colreduce_workspace_bytes(const tb200_group_desc *desc);
int tb200_colreduce_compile(const tb200_group_desc *desc);
int tb200_colreduce_compiled(const tb200_group_desc *desc, const void *const *inputs, void *const *outputs,
                             void *workspace, size_t workspace_bytes, void *stream);
size_t tb200_colreduce_source(const tb200_group_desc *desc, char *buffer, size_t buffer_bytes);

/* ---- scans: running folds along or across the rows --------------------------------
 * y = the running fold of x: every element of the result is the fold of the elements up to and
 * including its own position (Julia's `cumsum`, `cumprod`, `accumulate(max, ...)`, and `accumulate` by a
 * `GenericFold`), forward or from the far end (`reverse`: the derivative of a cumulative sum scans
 * backwards).  Replaces the kernels the reference generates for `:scan` groups
 * (ext/cuTileExt/build.jl:715-760), on the folds its scan tests exercise (test/cuda/scans.jl:12-22):
 *   SUM, PROD, MAX, MIN   the builtin folds (src/Compiler/IR/folds.jl:66-89)
 *   AFFINE                h = a h_prev + b from pairs (a, b) = (x, x2), starting from h = 0: the
 *                         `GenericFold` recurrence of src/Compiler/IR/folds.jl:279-288 and
 *                         test/fixtures/programs.jl:51-54 (combine ((a1,b1),(a2,b2)) = (a2 a1, a2 b1 + b2),
 *                         observe = last)
 *   VARIANCE              the running population variance by Welford's state merged Chan's way
 *                         (test/fixtures/programs.jl:44)
 * x, y are Julia (n, rows) matrices, memory [rows][n] with row pitches ld_* (elements); `across` = 0 scans
 * along each row (Julia dims = 1, the contiguous axis), 1 scans across the rows (dims = 2), one scan per
 * column; `batch` such matrices lie stride_* elements apart (a scan along the middle axis of a 3-axis
 * array is `across` over a batch).  Float32 or BFloat16 elements, Float32 states, results rounded once.
 * The order in which partial states are combined differs from a sequential sweep's (it is a tree over
 * threads), which rounds differently: the reference compares at rtol 1e-4 (test/cuda/scans.jl:27).
 * Nothing is kept between calls.  A scan across the rows of a matrix with few columns has only its columns
 * to spread over threads; given `workspace` (tb200_scan_workspace_bytes, 16-byte aligned) it is split into
 * slabs of rows instead: one launch folds every slab to its total, a second sweeps every slab again starting
 * from the totals before it (two reads and one write per element, in fixed order).  Without a workspace
 * (null) one thread walks each column. */
typedef enum tb200_scan_op {
    TB200_SCAN_SUM = 0, TB200_SCAN_PROD = 1, TB200_SCAN_MAX = 2, TB200_SCAN_MIN = 3,
    TB200_SCAN_AFFINE = 4, TB200_SCAN_VARIANCE = 5
} tb200_scan_op;
typedef struct tb200_scan_desc {
    int64_t n, rows;
    int64_t ld_x, ld_x2, ld_y;
    int64_t batch;                       /* 0 or 1 = one matrix */
    int64_t stride_x, stride_x2, stride_y;
    int op;                              /* tb200_scan_op */
    int across;
    int reverse;
    int dtype;
    void *workspace;                     /* optional, for `across` */
    size_t workspace_bytes;
} tb200_scan_desc;
size_t tb200_scan_workspace_bytes(const tb200_scan_desc *desc);
int tb200_scan(const tb200_scan_desc *desc, const void *x, const void *x2, void *y, void *stream);

/* ---- recurrences whose step is a map ------------------------------------------------
 * The `:recurrence` groups of the reference (src/Compiler/Implement/groups.jl:29-47; its kernel:
 * ext/cuTileExt/build.jl:772-835, a block per tile of the parallel axes stepping along the states' axis, the
 * states held in tiles) whose step computes every member element by element: states carried from step to step
 * (several, each assigned at once from the values before the step, so states may cross or lag:
 * test/runtime/recurrences.jl:190-196), members stored at every step, the states as the steps leave them --
 * h = tanh.(a .* h .+ x), exponential averages, gates that are maps of the step's inputs.  A step that contracts
 * over the state (a matrix times the hidden state) is not a map and is not taken here: DeltaNet's kernels and the
 * scans are the other recurrence kernels of this library.
 *
 * `body` is a group descriptor over (n, steps): n positions that do not interact (the parallel axes, collapsed),
 * `rows` = steps.  Terms are evaluated at every step in order; TB200_T_STATE reads a state before the step,
 * TB200_T_LOAD of a full input reads the step's row, of an `along` input a per-position constant, of a per-row
 * input the step's scalar; TB200_T_ROW_INDEX is the step.  No folds.  Outputs: from = 0, the term at every
 * step ((n, steps), row pitch ld); from = 3, state `index` after the last step (n values).  state k starts from
 * input `start` (shape along, or scalar) and is `next` (a term) after each step; `reverse` walks the steps from the
 * last.  One thread owns a position; eight steps' loads are issued ahead of the arithmetic.  Compiled by NVRTC on
 * first use and cached (TB200_ERR_UNSUPPORTED without NVRTC).  No workspace. */
#define TB200_RECURRENCE_MAX_STATES 4
typedef struct tb200_state { int start, next; } tb200_state;
typedef struct tb200_recurrence_desc {
    tb200_group_desc body;
    int n_states;
    tb200_state states[TB200_RECURRENCE_MAX_STATES];
    int reverse;
} tb200_recurrence_desc;
int tb200_recurrence_compile(const tb200_recurrence_desc *desc);
size_t tb200_recurrence_source(const tb200_recurrence_desc *desc, char *buffer, size_t buffer_bytes);
int tb200_recurrence_compiled(const tb200_recurrence_desc *desc, const void *const *inputs, void *const *outputs,
                              void *stream);

/* ---- data-parallel update: gradient sum + SGD step in one kernel over NVLink -----
 * The exchange of a data-parallel training step (the reference spells it `r .+ s` over the devices'
 * gradients followed by the update on each, realised by peer copies and sums:
 * src/Compiler/plan/devices.jl:7-11, test/fixtures/devices.jl `shards_sgd!`; replicas equal after
 * every step is its stated property).  Every rank calls tb200_dp_update at the same point of its
 * step with the same `count`, `alpha` and `blocks`.  Rank r sums the replicas' gradients over the
 * r-th slice of the range, forms params + alpha * sum once (Float32 arithmetic, gradients' sum and
 * the result rounded to BFloat16) and writes the result into every replica's `params`; the call
 * returns (in stream order) when every replica's `params` range is complete.  The replicas are
 * bit-equal by construction.  The gradient buffers are only read.
 *
 * grads[i], params[i], signals[i]: rank i's arrays as mapped into THIS process (peer-accessible
 * memory, e.g. a symmetric allocation; entry `rank` is the local one), 16-byte aligned.  With
 * grads_multicast / params_multicast (the same two ranges through an NVLink multicast mapping) the
 * sum is taken by the NVSwitch (multimem.ld_reduce) and the result broadcast by it (multimem.st);
 * NULL = plain loads from and stores to each peer.  signals[i]: tb200_dp_signal_bytes bytes,
 * zero before the first call, never touched by the caller afterwards.  state: local device memory,
 * tb200_dp_state_bytes bytes, zero before the first call.  Two calls that share signals or state
 * must not overlap on the GPU.  Ranks wait for one another inside the kernel; each wait gives up
 * after two seconds (a rank that never arrives) and tb200_dp_error then reports a non-zero code.
 * No allocation, no host synchronisation: the call can be captured, provided every rank replays it
 * the same number of times. */
typedef struct tb200_dp_desc {
    int rank, world;             /* world <= 16 */
    int blocks;                  /* thread blocks (SMs) the kernel occupies; 0 = 8; the same on every rank */
    int dtype;                   /* TB200_BF16 */
    int64_t count;               /* elements in the range, a multiple of 8 */
    float alpha;                 /* -rate */
    const void *grads[16];
    void *params[16];
    void *signals[16];
    const void *grads_multicast;
    void *params_multicast;
    void *state;
} tb200_dp_desc;
size_t tb200_dp_signal_bytes(void);
size_t tb200_dp_state_bytes(void);
int tb200_dp_update(const tb200_dp_desc *desc, void *stream);
/* As tb200_device_error, for tb200_dp_update: 0, or 1 + 16 * rank + peer of the first wait that gave up. */
int tb200_dp_error(void);

/* ---- pointwise maps and folds over other axes -------------------------------
 * These replace the generated `:pointwise` kernels (ext/cuTileExt/build.jl:3-10)
 * and the full / partial folds with their merge launches
 * (ext/cuTileExt/build.jl:560-705) for the loss, bias-gradient and update
 * groups of a training step (examples/mlp.jl:28-35). */

/* Clears a workspace (the squared-error ticket must start at zero; every call
 * leaves it zero again).  No reference counterpart. */
int tb200_workspace_clear(void *workspace, size_t workspace_bytes, void *stream);

size_t tb200_squared_error_workspace_bytes(void);

/* loss[0] = scale * sum((a - b)^2) (b NULL: sum(a^2), the README's
 * sum(abs2, ...)), and, when grad is not NULL, the loss's pullback
 * grad = grad_scale * 2 (a - b), times (1 - a^2) when through_tanh (a is a
 * tanh's output: src/Compiler/program/differentiate.jl:127, 134).  The sum is
 * merged in a fixed order.  workspace: tb200_squared_error_workspace_bytes
 * bytes, cleared once before its first use. */
int tb200_squared_error(const void *a, const void *b, void *grad, float *loss, int64_t count,
                        float scale, float grad_scale, int through_tanh, int dtype, void *workspace,
                        size_t workspace_bytes, void *stream);

size_t tb200_colsum_workspace_bytes(int64_t rows, int64_t n);

/* out[j] = scale * sum over rows of x[r][j]: the bias gradient, a fold over the
 * axis that is not contiguous (the reference's partial folds + merge,
 * ext/cuTileExt/emit.jl:744-753).  Float32 accumulation, fixed order. */
int tb200_colsum(const void *x, void *out, int64_t rows, int64_t n, int64_t ld, float scale,
                 int dtype, void *workspace, size_t workspace_bytes, void *stream);

/* y[i] += alpha * x[i]: the update w .- rate .* dw (examples/mlp.jl:32-35).
 * 128-bit accesses when y and x are both 16-byte aligned; a view that starts at
 * an odd element runs one element a thread. */
int tb200_axpy(void *y, const void *x, float alpha, int64_t count, int y_dtype, int x_dtype,
               void *stream);

#ifdef __cplusplus
}
#endif
#endif /* TEMPEST_B200_H */
