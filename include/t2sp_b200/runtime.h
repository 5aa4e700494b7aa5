/* C ABI of libt2sp_b200.so: the B200 replacement for the host interface and device
 * runtime that T2SP generates for its dense-tensor kernels.
 *
 * What it replaces in the reference:
 *   - the generated host functions `int <k>(halide_buffer_t*...)`
 *     (emitter Halide/src/CodeGen_C.cpp:1712-1738,2746-2818; checked-in example
 *     t2s/peppers/blas/level3/syrk/release/s10/syrk-interface.{h,cpp}),
 *   - the AOT device runtime they call (t2s/src/AOT-OpenCL-Runtime.{h,cpp}),
 *   - the generated device kernels (e.g. t2s/tests/performance/gemm/bitstream/a10/a.cl).
 *
 * Conventions kept from the reference: inputs first, output last; return 0 on success,
 * otherwise the negative halide_error_code_t that the matching halide_error_* reporter
 * returns (HalideRuntime.h:957-1143); buffers are caller-owned; dim 0 is innermost with
 * stride 1; a buffer with host==NULL and device==0 is a bounds query and gets its shape
 * filled in. Differences: calls are repeatable and thread-safe, nothing ever exits the
 * process, and there is no CPU fallback: without a CUDA device every compute entry fails
 * with halide_error_code_device_interface_no_device.
 */
#ifndef T2SP_B200_RUNTIME_H
#define T2SP_B200_RUNTIME_H

#include "abi.h"

#ifdef __cplusplus
extern "C" {
#endif

#ifdef T2SP_B200_OWN_HALIDE_ABI
/* halide_error_code_t (HalideRuntime.h:957-1143): the codes this library and its error reporters return. */
enum halide_error_code_t {
    halide_error_code_success = 0,
    halide_error_code_generic_error = -1,
    halide_error_code_explicit_bounds_too_small = -2,
    halide_error_code_bad_type = -3,
    halide_error_code_access_out_of_bounds = -4,
    halide_error_code_buffer_allocation_too_large = -5,
    halide_error_code_buffer_extents_too_large = -6,
    halide_error_code_constraints_make_required_region_smaller = -7,
    halide_error_code_constraint_violated = -8,
    halide_error_code_param_too_small = -9,
    halide_error_code_param_too_large = -10,
    halide_error_code_out_of_memory = -11,
    halide_error_code_buffer_argument_is_null = -12,
    halide_error_code_debug_to_file_failed = -13,
    halide_error_code_copy_to_host_failed = -14,
    halide_error_code_copy_to_device_failed = -15,
    halide_error_code_device_malloc_failed = -16,
    halide_error_code_device_sync_failed = -17,
    halide_error_code_device_free_failed = -18,
    halide_error_code_no_device_interface = -19,
    halide_error_code_device_run_failed = -23,
    halide_error_code_unaligned_host_ptr = -24,
    halide_error_code_bad_fold = -25,
    halide_error_code_fold_factor_too_small = -26,
    halide_error_code_requirement_failed = -27,
    halide_error_code_buffer_extents_negative = -28,
    halide_error_code_failed_to_upgrade_buffer_t = -29,
    halide_error_code_failed_to_downgrade_buffer_t = -30,
    halide_error_code_specialize_fail = -31,
    halide_error_code_device_wrap_native_failed = -32,
    halide_error_code_host_is_null = -34,
    halide_error_code_bad_extern_fold = -35,
    halide_error_code_device_interface_no_device = -36,
    halide_error_code_host_and_device_dirty = -37,
    halide_error_code_buffer_is_null = -38,
    halide_error_code_device_buffer_copy_failed = -39,
    halide_error_code_bad_dimensions = -43,
    halide_error_code_integer_division_by_zero = -44
};
#endif

/* ---- element types accepted --------------------------------------------------------
 * fp32 in / fp32 out (the reference's only type: type word 73730, syrk-interface.cpp:149);
 * additionally bf16 or f16 in / fp32 out and int8 in / int32 out for GEMM.            */

/* How fp32 inputs are multiplied on the tensor cores. */
enum t2sp_precision {
    T2SP_PRECISION_DEFAULT = 0, /* $T2SP_B200_PRECISION if set, else TF32X3 */
    T2SP_PRECISION_TF32X3 = 1,  /* three TF32 MMAs per product, ~fp32 accuracy */
    T2SP_PRECISION_TF32 = 2     /* one TF32 MMA per product: 10-bit mantissas, ~1e-3 accuracy, about 3x faster */
};

/* ---- GEMM:  C[i,j] = sum_k A[i,k] * B[k,j]          (t2s/tests/performance/gemm/gemm.cpp:30-63)
 * A: 2-D (K_tot, I_tot), B: 2-D (J_tot, K_tot)                                (gemm.cpp:58-59)
 * C: layout 0 = 2-D (J_tot, I_tot)                               (gemm.cpp:89, gemm-run-gpu.cpp:58)
 *    layout 1 = 6-D (JJJ, III, JJ, II, J, I), element (jjj,iii,jj,ii,j,i) holds
 *               C[iii + III*ii + III*II*i, jjj + JJJ*jj + JJJ*JJ*j]    (gemm-run-fpga.cpp:69,80-85)
 * With desc == NULL the layout is taken from C->dimensions and, for 6-D, the tile extents
 * from C's own extents.                                                                */
typedef struct t2sp_gemm_desc {
    int32_t layout;
    int32_t JJJ, III, JJ, II; /* layout 1: inner tile extents (0 = read them from C) */
    int32_t precision;        /* enum t2sp_precision */
    int32_t trans_b;          /* 1: B is stored transposed, 2-D (K_tot, J_tot) with k innermost */
    int32_t trans_a;          /* 1: A is stored transposed, 2-D (I_tot, K_tot) with i innermost (fp32 only;
                                 a transposed copy is made on the device) */
    int32_t scale;            /* 1: C = alpha * A x B + beta * C (fp32 output, layout 0); C is then read too */
    float alpha, beta;
} t2sp_gemm_desc;
int t2sp_b200_gemm(halide_buffer_t *A, halide_buffer_t *B, halide_buffer_t *C, const t2sp_gemm_desc *desc);

/* BLAS-style front of the same kernel, the counterpart of the reference's PEPPERS wrapper
 * `sgemm(transa, transb, m, n, k, alpha, a, lda, b, ldb, beta, c, ldc)`
 * (t2s/peppers/blas/level3/gemm/release/a10/blas-gemm.{h,cpp}, driver sgemm-run-fpga.cpp):
 * row-major host arrays, op(A) is m x k, op(B) is k x n, C = alpha*op(A)*op(B) + beta*C.
 * 'N'/'n' = as stored, anything else = transposed. A leading dimension <= 0 means dense, which is
 * what the reference driver passes (it calls with lda = ldb = ldc = 0). Returns a halide error code. */
int t2sp_b200_sgemm(char transa, char transb, int m, int n, int k, float alpha, const float *a, int lda,
                    const float *b, int ldb, float beta, float *c, int ldc);

/* ---- 2-D convolution, stride 1, input already enlarged by KX-1 / KY-1
 *                                                     (t2s/tests/performance/conv/conv.cpp:30-65)
 * I: 2-D (CI*N, IY*IX)    element (ci + CI*n, iy + IY*ix)                     (conv.cpp:52)
 * K: 2-D (CO*KX, CI*KY)   element (co + CO*kx, ci + CI*ky)                    (conv.cpp:53)
 * O: layout 0 = 2-D (CO*N, OY*OX)  element (co + CO*n, oy + OY*ox)            (conv.cpp:54)
 *    layout 1 = 10-D (COOO,YYY,XXX,COO,YY,XX,Y,X,CO,N)              (conv-run-fpga.cpp:68,73-93)
 * The flattened 2-D buffers cannot be un-flattened without CI, CO, KY, KX, OY, OX, which
 * the reference bakes into the generated code from const-parameters.h; here they arrive
 * in the descriptor. N is read from the buffers.                                       */
typedef struct t2sp_conv_desc {
    int32_t layout;
    int32_t CI, CO, KY, KX, OY, OX;              /* totals */
    int32_t COOO, YYY, XXX, COO, YY, XX, Y, X;   /* layout 1 tile extents (CO outer and N come from O) */
    int32_t precision;
} t2sp_conv_desc;
int t2sp_b200_conv(halide_buffer_t *I, halide_buffer_t *K, halide_buffer_t *O, const t2sp_conv_desc *desc);

/* ---- capsule convolution: per output pose V[my,mx] = sum W[my,mk] * P[mk,mx] over
 * (mk, ci, ky, kx), input position (s*oy+ky, s*ox+kx)   (t2s/tests/performance/capsule/capsule.cpp:28-66)
 * P: 2-D (CI*MK*MX*NN, IY*IX*N)   element (ci + CI*mk + CI*MK*mx + CI*MK*MX*nn, iy + IY*ix + IY*IX*n)
 * W: 2-D (CO*MY, CI*KY*KX*MK)     element (co + CO*my, cii + CII*ky + CII*KY*kx + CII*KY*KX*ci_o + CI*KY*KX*mk)
 * V: layout 0 = 2-D (CO*MY*MX*NN, OY*OX*N)                                 (capsule.cpp:52-54)
 *    layout 1 = 10-D (COOO,YYY_XXX,YY_XX,Y_X,MY,MX,COO,NN,CO,N), pixel slot
 *               p = yyy_xxx + YYY_XXX*yy_xx + YYY_XXX*YY_XX*y_x, oy = p % OY, ox = p / OY;
 *               slots with p >= OY*OX are written as 0        (capsule-run-fpga.cpp:73,78-104)
 * IY = s*OY + KY - s, IX likewise. The reference hard-codes s = 2 (capsule.cpp:40-41). */
typedef struct t2sp_capsule_desc {
    int32_t layout;
    int32_t CI, CII, CO, KY, KX, OY, OX, MY, MX, MK, NN, stride;
    int32_t COOO, YYY_XXX, YY_XX, Y_X, COO;      /* layout 1 tile extents */
    int32_t precision;
} t2sp_capsule_desc;
int t2sp_b200_capsule(halide_buffer_t *P, halide_buffer_t *W, halide_buffer_t *V, const t2sp_capsule_desc *desc);

/* N-D operands of the reference's oneAPI flow (spatial index innermost):
 *   conv:    I 4-D (IY, IX, CI, N), K 4-D (KY, KX, CI, CO), O 10-D as above
 *            (t2s/tests/correctness/oneapi-integration/oneapi-target-5-conv.cpp:58-62, -5-run.cpp:92-103)
 *   capsule: P 6-D (MK, MX, CI, IY, IX, N), W 6-D (MY, MK, CI, CO, KY, KX),
 *            V 9-D (COOO, YYY_XXX, YY_XX, Y_X, MY, MX, COO, CO, N)
 *            (oneapi-target-6-capsule.cpp:57-61, -6-run.cpp:92-99)
 * Every constant comes from the extents (capsule: stride 2 as in the reference, or 1, whichever
 * fits V's pixel slots); `precision` is a t2sp_precision. Bounds queries are not answered. */
/* SYRK as the PEPPERS BLAS layer's generated interface takes it
 * (t2s/peppers/blas/level3/syrk/release/s10/syrk-interface.h:12, t2s/tests/performance/syrk/syrk.cpp:52-73):
 * A 2-D (K, N), symmetric C 2-D (N, N), O 6-D (III, III, II, II, I+1, >= I/2) with N = III*II*I;
 * O(jjj,iii,jj,ii,j,i) = Alpha * sum_k A(k,r) A(k,c) + Beta * C(c,r), where for i >= j
 * (r, c) = (N-1-ti, N-1-tj) and otherwise (r, c) = (ti, tj - III*II),
 * ti = iii + III*ii + III*II*i, tj = jjj + III*jj + III*II*j. OpA is ignored, as in the specification. */
int t2sp_b200_syrk(int32_t OpA, float Alpha, float Beta, halide_buffer_t *A, halide_buffer_t *C, halide_buffer_t *O);

/* GER as the design's generated interface takes it (t2s/tests/performance/ger/ger.cpp:34-62,112;
 * driver ger-run-fpga.cpp:50-82): A 2-D (TK, TI), X 1-D (TI), Y 1-D (TK), O 6-D (KKK, III, II, KK, K, I)
 * with TK = KKK*KK*K and TI = III*II*I; O(kkk,iii,ii,kk,k,i) = A(tk, ti) + X(ti) * Y(tk),
 * ti = iii + III*ii + III*II*i, tk = kkk + KKK*kk + KKK*KK*k (one fp32 multiply and one add, unfused). */
int t2sp_b200_ger(halide_buffer_t *A, halide_buffer_t *X, halide_buffer_t *Y, halide_buffer_t *O);

int t2sp_b200_conv_nd(halide_buffer_t *I, halide_buffer_t *K, halide_buffer_t *O, int precision);
int t2sp_b200_capsule_nd(halide_buffer_t *P, halide_buffer_t *W, halide_buffer_t *V, int precision);

/* ---- TTM:  c(i,j,k) = sum_l a(l,i,j) * b(l,k)   (t2s/tests/correctness/buffer/tmm_small.cpp:46-64,
 *                                                  golden t2s/tests/correctness/util/util.h:428-441)
 * a: 3-D (L,I,J), b: 2-D (L,K)
 * c: layout 0 = 3-D (I,J,K)
 *    layout 1 = 9-D (JJ,KK,II,KKK,JJJ,III,OK,OJ,OI) with i = iii + III*ii + III*II*oi,
 *               j = jjj + JJJ*jj + JJJ*JJ*oj, k = kkk + KKK*kk + KKK*KK*ok  (tmm_small.cpp:116-129) */
typedef struct t2sp_ttm_desc {
    int32_t layout;
    int32_t precision;
} t2sp_ttm_desc;
int t2sp_b200_ttm(halide_buffer_t *a, halide_buffer_t *b, halide_buffer_t *c, const t2sp_ttm_desc *desc);

/* ---- MTTKRP:  d(i,r) = sum_k ( sum_l a(l,i,k) * c(l,r) ) * b(k,r)
 *                                   (golden only: t2s/tests/correctness/util/util.h:464-481, with
 *                                    its outer loop bound `i < K` read as `i < I`)
 * a: 3-D (L,I,K), b: 2-D (K,R), c: 2-D (L,R), d: 2-D (I,R). Argument order follows the
 * golden helper: (a, b, c, d). The Khatri-Rao product of b and c is formed tile by tile
 * in shared memory and never written to global memory.                                 */
typedef struct t2sp_mttkrp_desc {
    int32_t precision;
    int32_t splits; /* split factor over the (l,k) contraction; 0 = choose */
} t2sp_mttkrp_desc;
int t2sp_b200_mttkrp(halide_buffer_t *a, halide_buffer_t *b, halide_buffer_t *c, halide_buffer_t *d,
                     const t2sp_mttkrp_desc *desc);

/* ---- MTTKRP without any allocation ---------------------------------------------------
 * No counterpart in the reference (its runtime allocates per call,
 * syrk-interface.cpp:951-966). For callers that must not allocate device memory while they
 * run: services with a fixed memory pool, loops that cannot take cudaMalloc's implicit device
 * synchronisation, code under a framework allocator that owns all of HBM.
 * Same contraction and layouts as t2sp_b200_mttkrp, but every pointer is a CUDA device
 * pointer (element strides given explicitly, innermost stride 1), and the split partial
 * sums use a fixed array of T2SP_B200_NOALLOC_SCRATCH_BYTES inside the loaded module instead
 * of the library's allocator. The call performs no cudaMalloc/cudaFree and no host staging.
 *  - limit: 4*I*R bytes (one partial slab) must fit in the array, else
 *    halide_error_code_buffer_allocation_too_large; R <= 128; `a` and `c` 16-byte aligned with
 *    strides that are multiples of 4 elements.
 *  - every GPU that loads the library holds the array until the process exits; all calls on
 *    a device share it (contents of the previous call remain; nothing has to be cleared
 *    because each split rewrites its slab), so calls that overlap on the GPU race.
 *  - the first call on each device looks up the array's address; make it outside stream capture.
 *  - sync != 0: waits for `cuda_stream` and returns the kernels' status; sync == 0: returns
 *    after enqueueing on `cuda_stream` (NULL = default stream). A status that a sync == 0 call's
 *    kernels raise (a bounded wait that ran out) is reported, and cleared, by the next sync != 0
 *    call on that device.                                                                  */
#define T2SP_B200_NOALLOC_SCRATCH_BYTES (16u << 20)
int t2sp_b200_mttkrp_noalloc(const float *a, int64_t a_stride_i, int64_t a_stride_k, const float *b,
                             int64_t b_stride_r, const float *c, int64_t c_stride_r, float *d, int64_t d_stride_r,
                             int32_t L, int32_t I, int32_t K, int32_t R, void *cuda_stream, int32_t sync);

/* ---- device residency --------------------------------------------------------------
 * Counterpart of halide_device_malloc / halide_copy_to_device / halide_copy_to_host /
 * halide_device_free in t2s/src/AOT-OpenCL-Runtime.cpp:74-117,402-441, and of
 * halide_cuda_wrap_device_ptr (Halide/src/runtime/HalideRuntimeCuda.h:45-60).
 * A buffer whose `device` field is non-zero and whose device_interface is
 * t2sp_b200_device_interface() is read from / written to device memory directly:
 * inputs are copied from `host` only if no device copy exists or host_dirty is set;
 * outputs stay on the device (device_dirty is set) when the output buffer has a device
 * allocation, otherwise they are copied to `host` and host_dirty is set.             */
/* The interface is a full function table (HalideRuntime.h:713-738): Halide::Runtime::Buffer's
 * copy_to_host(), device_free(), crops, slices and destructor work on buffers this library filled.
 * Host threads: each thread works on a stream, timing events and a kernel status word of its own
 * (or on the stream given with t2sp_b200_set_stream); cached device blocks that change streams are
 * ordered by events, so threads may call concurrently. */
const struct halide_device_interface_t *t2sp_b200_device_interface(void);
int t2sp_b200_device_malloc(halide_buffer_t *buf);
int t2sp_b200_device_free(halide_buffer_t *buf);
int t2sp_b200_copy_to_device(halide_buffer_t *buf);
int t2sp_b200_copy_to_host(halide_buffer_t *buf);
int t2sp_b200_wrap_device_ptr(halide_buffer_t *buf, uint64_t device_ptr);
int t2sp_b200_detach_device_ptr(halide_buffer_t *buf);

/* ---- several GPUs of one box: one process (or host thread) per GPU -----------------------
 * No counterpart in the reference, which drives one device (AOT-OpenCL-Runtime.cpp:186-213).
 * Every rank calls the same entry with its rank and the world size, on FULL-SIZE buffers (host
 * or device-resident); the entry works on this rank's slab of them, which is a view (shifted
 * base address, unchanged strides), never a copy:
 *   gemm     columns of B and C (A replicated; plain 2-D output layout)
 *   conv     batch items n of I and O (weights replicated; plain layout)
 *   capsule  batch items n of P and V (weights replicated; plain layout)
 *   ttm      index j of a(l,i,j) and c(i,j,k) (b replicated; plain layout)
 *   mttkrp   index k of a(l,i,k) and b(k,r), i.e. the contraction: d_partial is this rank's
 *            full-size partial result, to be summed over the ranks
 * Slabs are contiguous and near-equal (t2sp_b200_split_range); a rank whose slab is empty does
 * nothing and returns 0. The contractions themselves exchange nothing between GPUs. */
void t2sp_b200_split_range(int64_t total, int32_t world, int32_t rank, int64_t *lo, int64_t *hi);
/* dst (with room for src->dimensions entries in dst_dims) becomes the view of src restricted, in
 * dimension `dim`, to this rank's share of its extent / unit groups of `unit` consecutive indices. */
int t2sp_b200_shard_view(const halide_buffer_t *src, int32_t dim, int32_t unit, int32_t rank, int32_t world,
                         halide_buffer_t *dst, halide_dimension_t *dst_dims);
int t2sp_b200_gemm_shard(halide_buffer_t *A, halide_buffer_t *B, halide_buffer_t *C, const t2sp_gemm_desc *desc,
                         int32_t rank, int32_t world);
int t2sp_b200_conv_shard(halide_buffer_t *I, halide_buffer_t *K, halide_buffer_t *O, const t2sp_conv_desc *desc,
                         int32_t rank, int32_t world);
int t2sp_b200_capsule_shard(halide_buffer_t *P, halide_buffer_t *W, halide_buffer_t *V, const t2sp_capsule_desc *desc,
                            int32_t rank, int32_t world);
int t2sp_b200_ttm_shard(halide_buffer_t *a, halide_buffer_t *b, halide_buffer_t *c, const t2sp_ttm_desc *desc,
                        int32_t rank, int32_t world);
int t2sp_b200_mttkrp_shard(halide_buffer_t *a, halide_buffer_t *b, halide_buffer_t *c, halide_buffer_t *d_partial,
                           const t2sp_mttkrp_desc *desc, int32_t rank, int32_t world);
/* The exchange steps, for callers that want a result on every GPU; NCCL over NVLink, enqueued on the
 * calling thread's stream. libnccl.so.2 is looked up on the first of these calls. `comm` is an
 * ncclComm_t: the caller's own, or one made here (rank 0 obtains the 128-byte id and hands it to the
 * other ranks by whatever means the host program has; every rank then calls t2sp_b200_comm_init with
 * its device selected by t2sp_b200_set_device).
 *   gather_columns   C (2-D, device-resident, full size on every rank, each rank's slab computed):
 *                    afterwards every rank holds all columns.
 *   reduce_partials  d (2-D fp32, device-resident): the sum over the ranks, in place on every rank;
 *                    ordered != 0 adds the partials in rank order (bitwise reproducible), else ncclAllReduce.
 *   broadcast        the buffer's device copy on `root` replaces everyone's (replicating an operand). */
int t2sp_b200_nccl_unique_id(void *id_bytes, int32_t size); /* size >= 128 */
int t2sp_b200_comm_init(void **comm, int32_t world, const void *id_bytes, int32_t rank);
int t2sp_b200_comm_destroy(void *comm);
int t2sp_b200_gather_columns(halide_buffer_t *C, void *comm, int32_t rank, int32_t world);
int t2sp_b200_reduce_partials(halide_buffer_t *d, void *comm, int32_t rank, int32_t world, int32_t ordered);
int t2sp_b200_broadcast(halide_buffer_t *buf, void *comm, int32_t root);

/* ---- execution control -------------------------------------------------------------
 * Calls are synchronous by default, like the reference's (clFinish per call,
 * AOT-OpenCL-Runtime.cpp:312-358). */
int t2sp_b200_set_device(int ordinal);          /* CUDA device for the calling thread (default 0) */
int t2sp_b200_set_stream(void *cuda_stream);    /* stream for the calling thread; NULL = the thread's own library stream */
int t2sp_b200_set_async(int enable);            /* 1: calls on device-resident buffers return after enqueue */
int t2sp_b200_sync(void);                       /* wait for the thread's stream; reports kernel status */
void t2sp_b200_release(void);                   /* wait for the devices and free cached device allocations */
/* The T2SP_B200_* environment variables (and BITSTREAM) are read once, at the first call; this reads
 * them again. Not to be called while another thread is inside the library. */
void t2sp_b200_reload_env(void);
uint64_t t2sp_b200_kernel_launches(void);       /* kernels launched by this library since load */
/* Device time of the last synchronous call's kernels in nanoseconds, as the reference's
 * runtime records per kernel (AOT-OpenCL-Runtime.cpp:360-396). It is also written to
 * exec_time.txt in dirname($BITSTREAM) or to $T2SP_B200_EXEC_TIME_FILE when set.      */
double t2sp_b200_last_kernel_ns(void);
const char *t2sp_b200_version(void);
/* SM count and maximum SM clock (kHz) of the calling thread's device; 0 on success. */
int t2sp_b200_device_info(int *sm_count, int *sm_clock_khz);

#ifdef __cplusplus
}
#endif
#endif /* T2SP_B200_RUNTIME_H */
