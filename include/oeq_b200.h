/*
 * oeq_b200 -- C ABI of the B200 (sm_100a) tensor-product / graph-convolution kernels.
 *
 * This is the boundary that replaces the reference's pybind11 extension
 * `kernel_wrapper` (openequivariance/extension/kernel_wrapper.cpp:23-66).  Every
 * entry point takes plain pointers and sizes, returns an int status (0 = OK) and
 * never exits or throws across the boundary; oeq_last_error() gives the text of
 * the calling thread's last failure.  The library allocates no user-visible
 * memory: inputs, outputs and scratch are the caller's device buffers.  A handle
 * loads its kernels on first use and, for shared-weight 'uvw' problems, owns a
 * device copy of the weights in the tensor cores' operand layout (a few hundred
 * KB, allocated on first use, rewritten by every call): calls on one handle must
 * not run concurrently from several host threads or on several streams at once;
 * different handles are independent.  Launches are asynchronous on the stream that
 * is passed in (a cudaStream_t as void*), on the CUDA device that is current in
 * the calling thread.
 *
 * Data layout: row-major [rows][dim]; within a row the irreps are concatenated,
 * each as a [mul][2l+1] block.  Weights are in the kernel ("oeq") order defined
 * by the reference (openequivariance/implementations/ComputationSchedule.py:427-471).
 */
#ifndef OEQ_B200_H
#define OEQ_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
    OEQ_OK = 0,
    OEQ_ERR_INVALID = 1,     /* bad argument / malformed problem */
    OEQ_ERR_UNSUPPORTED = 2, /* well-formed problem outside the supported set */
    OEQ_ERR_COMPILE = 3,     /* run-time specialisation of a kernel failed */
    OEQ_ERR_CUDA = 4,        /* a CUDA runtime call failed */
    OEQ_ERR_DEVICE_WAIT = 5  /* a kernel gave up on a bounded wait */
};

enum { OEQ_MODE_UVU = 0, OEQ_MODE_UVW = 1 };
enum { OEQ_F32 = 0, OEQ_F64 = 1 };

/* One entry of an Irreps: mul copies of (l, parity).
 * Reference: openequivariance/implementations/e3nn_lite.py:157-188. */
typedef struct oeq_irrep {
    int32_t mul;
    int32_t l;
    int32_t parity; /* +1 or -1 */
} oeq_irrep;

/* One instruction with its normalised path weight and the nonzeros of its real
 * Clebsch-Gordan tensor C[i][j][k] (without the path weight).
 * Reference: openequivariance/implementations/e3nn_lite.py:355-362 (Instruction),
 * openequivariance/implementations/ComputationSchedule.py:52-66 (CGTensor). */
typedef struct oeq_instruction {
    int32_t i_in1, i_in2, i_out;
    int32_t mode; /* OEQ_MODE_UVU or OEQ_MODE_UVW */
    double path_weight;
    int32_t cg_nnz;
    const int32_t* cg_i;
    const int32_t* cg_j;
    const int32_t* cg_k;
    const double* cg_value;
} oeq_instruction;

/* Reference: openequivariance/implementations/e3nn_lite.py:365-523 (TPProblem). */
typedef struct oeq_problem_desc {
    int32_t n_in1, n_in2, n_out, n_instr;
    const oeq_irrep* in1;
    const oeq_irrep* in2;
    const oeq_irrep* out;
    const oeq_instruction* instr;
    int32_t dtype;          /* OEQ_F32 or OEQ_F64; irreps and weights share it */
    int32_t shared_weights; /* 1: W is [weight_numel]; 0: W is [rows][weight_numel];
                               2 ('uvu' convolution only): there is no weight array, every weight is 1 -- W and dW
                               may be NULL and are not touched (used for the edge sum in front of a shared dense
                               contraction; no counterpart in the reference) */
} oeq_problem_desc;

typedef struct oeq_tp oeq_tp;
typedef struct oeq_conv oeq_conv;

const char* oeq_version(void);
const char* oeq_last_error(void);

/* Where the kernel headers live and where compiled kernels are cached.  Defaults:
 * "<directory of this library>/csrc" and "<directory of this library>/_kcache". */
int oeq_set_kernel_dir(const char* path);
int oeq_set_cache_dir(const char* path);

/* Specialise (or fetch from the cache) the kernels of a problem without touching a
 * GPU.  kinds is a bit mask: 1 batch TP, 2 deterministic conv, 4 atomic conv, 8 (with 2 or 4) also the
 * second-derivative kernels of that convolution. */
int oeq_precompile(const oeq_problem_desc* desc, int kinds);

/* ---- batch tensor product --------------------------------------------------------
 * Replaces JITTPImpl (openequivariance/extension/tensorproducts.hpp:50-98). */
int oeq_tp_create(const oeq_problem_desc* desc, oeq_tp** out);
int oeq_tp_destroy(oeq_tp* h);
int64_t oeq_tp_weight_numel(const oeq_tp* h);

/* Z[b] = TP(X[b], Y[b], W[b] or W).  Replaces JITTPImpl::exec_tensor_product
 * (tensorproducts.hpp:76-85).  Every element of Z is written. */
int oeq_tp_forward(oeq_tp* h, int64_t batch, const void* X, const void* Y, const void* W, void* Z,
                   void* stream);

/* Scratch needed by oeq_tp_backward for `batch` rows (0 unless weights are shared). */
size_t oeq_tp_workspace_bytes(const oeq_tp* h, int64_t batch);

/* dX, dY, dW from X, Y, W, dZ.  Replaces JITTPImpl::backward (tensorproducts.hpp:87-95).
 * With shared weights dW is the sum over the batch, accumulated in a fixed order. */
int oeq_tp_backward(oeq_tp* h, int64_t batch, const void* X, const void* Y, const void* W, const void* dZ,
                    void* dX, void* dY, void* dW, void* workspace, size_t workspace_bytes, void* stream);

/* Same result as oeq_tp_backward for a shared-weight problem, for callers that may not allocate device
 * memory and so cannot hand over scratch: code running where the surrounding framework owns all
 * allocation (a memory pool that must not be bypassed, a real-time loop after its set-up phase).
 * It has no counterpart in the reference.  The partial weight gradients go to a fixed 8 MiB array
 * inside the library image (held by every GPU that loads the library); the launch is narrowed until
 * its partials fit, and a weight tensor larger than the array is refused with OEQ_ERR_UNSUPPORTED.
 * The call itself makes no cudaMalloc / cudaFree; the first call on a device (and the first call on
 * a handle) does one-time set-up -- the array's address is looked up (under a lock, so host threads
 * may race to it), the kernels are loaded -- so make that call before any stream capture.  All calls
 * share the array, which keeps whatever the last call left; every call rewrites the part it reads,
 * but two calls that overlap on the GPU race.  'uvw' problems always take the FMA kernels here (the
 * tensor-core kernels of oeq_tp_backward need packed weight copies that the library would have to
 * allocate), so expect that pass to be several times slower than oeq_tp_backward for them.  A
 * bounded wait that runs out is recorded only if the handle already owns a status word (any earlier
 * oeq_tp_forward / oeq_tp_backward creates it). */
int oeq_tp_backward_noalloc(oeq_tp* h, int64_t batch, const void* X, const void* Y, const void* W, const void* dZ,
                            void* dX, void* dY, void* dW, void* stream);

/* Second derivatives in one pass.  With dX, dY, dW the results of oeq_tp_backward for (X, Y, W, dZ), this gives the
 * gradient of <EX, dX> + <EY, dY> + <EW, dW> with respect to X, Y, W and dZ (GX, GY, GW, GdZ; every element written).
 * The reference composes this from four backward and three forward launches
 * (openequivariance/implementations/TensorProductBase.py:284-296); this entry point reads a row's seven arrays once.
 * Available for 'uvu' problems with per-row weights and a second input of multiplicity 1 whose rows fit two
 * shared-memory stages (oeq_tp_has_double_backward); otherwise OEQ_ERR_UNSUPPORTED, and the caller composes it. */
int oeq_tp_has_double_backward(const oeq_tp* h);
int oeq_tp_double_backward(oeq_tp* h, int64_t batch, const void* X, const void* Y, const void* W, const void* dZ,
                           const void* EX, const void* EY, const void* EW, void* GX, void* GY, void* GW, void* GdZ,
                           void* stream);

/* Reads the handle's device status word (synchronises the stream it last ran on):
 * OEQ_OK, or OEQ_ERR_DEVICE_WAIT if a kernel abandoned a bounded wait. */
int oeq_tp_check(oeq_tp* h);

/* ---- fused graph convolution -------------------------------------------------------
 * Z[n] = sum over edges e with rows[e] == n of TP(X[cols[e]], Y[e], W[e]).
 * Replaces JITConvImpl (openequivariance/extension/convolution.hpp:94-176).
 * deterministic != 0: edges must be sorted by receiver (rows); the backward pass
 * needs perm with perm[k] = position of the k-th edge in (sender, receiver) order.
 * rows/cols/perm are int64. */
int oeq_conv_create(const oeq_problem_desc* desc, int deterministic, oeq_conv** out);
int oeq_conv_destroy(oeq_conv* h);
/* Preferred scratch for oeq_conv_backward (the forward pass needs none).  Deterministic variant: one dX
 * row per edge, capped at 8 GiB (environment OEQ_B200_BWD_SCRATCH_MB); the backward pass then walks the
 * edges in receiver order, keeps the receiver's dZ slice on chip, writes each edge's dX row to the scratch
 * and sums the rows per sender in sender_perm order (in blocks of edges when the scratch is smaller than
 * the edge list).  The scratch is optional: with a null or small workspace the pass runs the sender-order
 * kernel, which needs none and gives the same results up to summation order.  Atomic variant: 0.
 * (The reference sizes a workspace for its fix-up pass here: LoopUnrollConv.py:61-72.) */
size_t oeq_conv_workspace_bytes(const oeq_conv* h, int64_t nodes, int64_t edges);

/* Replaces JITConvImpl::exec_conv (convolution.hpp:121-147).  Every row of Z is written. */
int oeq_conv_forward(oeq_conv* h, int64_t nodes, int64_t edges, const void* X, const void* Y, const void* W,
                     const int64_t* rows, const int64_t* cols, void* Z, void* workspace,
                     size_t workspace_bytes, void* stream);

/* Replaces JITConvImpl::backward (convolution.hpp:149-173).  Every row of dX is written. */
int oeq_conv_backward(oeq_conv* h, int64_t nodes, int64_t edges, const void* X, const void* Y, const void* W,
                      const void* dZ, const int64_t* rows, const int64_t* cols, const int64_t* perm,
                      void* dX, void* dY, void* dW, void* workspace, size_t workspace_bytes, void* stream);

int oeq_conv_check(oeq_conv* h);

/* Number of kernels the most recent oeq_conv_backward on this handle launched: 1 for the sender-order kernel
 * and for the atomic receiver-order kernel; for the deterministic receiver-order pass the kernel that clears dX,
 * one launch per block of edges (each sums the previous block's rows as well when the blocks are pipelined)
 * and the row-sum launches.  Benchmarks report it; it has no counterpart in the reference. */
int oeq_conv_last_backward_launches(const oeq_conv* h);

/* Second derivatives of the convolution in two fused launches (plus the row sum of the deterministic variant).
 * With dX, dY, dW the results of oeq_conv_backward for the output gradient dZ, and EX [nodes, x_dim], EY [edges,
 * y_dim], EW [edges, weight_numel] cotangents of those three, this computes the gradients of
 * <EX, dX> + <EY, dY> + <EW, dW> with respect to X, Y, W and dZ: GX [nodes, x_dim], GY, GW (per edge) and GdZ
 * [nodes, z_dim].  The reference composes them from four backward and three forward launches of the same graph
 * (openequivariance/implementations/convolution/ConvolutionBase.py, double_backward of the registered op); here an
 * edge's rows and cotangent rows are staged once per launch.  rows/cols/perm as for oeq_conv_backward; the
 * deterministic variant needs scratch of oeq_conv_workspace_bytes (it returns OEQ_ERR_UNSUPPORTED without it, and the
 * caller composes the result from oeq_conv_forward / oeq_conv_backward instead).  The kernels are compiled at the
 * first call.  oeq_conv_has_double_backward: 1 when the problem qualifies (per-edge weights, one thread per
 * channel), else 0. */
int oeq_conv_has_double_backward(const oeq_conv* h);
int oeq_conv_double_backward(oeq_conv* h, int64_t nodes, int64_t edges, const void* X, const void* Y, const void* W,
                             const void* dZ, const void* EX, const void* EY, const void* EW, const int64_t* rows,
                             const int64_t* cols, const int64_t* sender_perm, void* GX, void* GY, void* GW, void* GdZ,
                             void* workspace, size_t workspace_bytes, void* stream);

/* Exercises the error path of the kernels' bounded waits without harming the device: one thread polls a barrier
 * that nothing completes `polls` times (at most 2^20), gives up, and the call reports what oeq_*_check would report,
 * OEQ_ERR_DEVICE_WAIT.  The context stays usable.  No counterpart in the reference (its kernels have no waits). */
int oeq_selftest_bounded_wait(int polls, void* stream);

/* Launch geometry of the most recent specialisation, for benchmarks and tests:
 * which = 0 forward, 1 backward.  Any output pointer may be NULL. */
int oeq_tp_launch_info(const oeq_tp* h, int which, int* threads, int* groups_per_cta, int* partitions,
                       int* stages, int* smem_bytes, int* registers);
int oeq_conv_launch_info(const oeq_conv* h, int which, int* threads, int* groups_per_cta, int* partitions,
                         int* stages, int* smem_bytes, int* registers);

#ifdef __cplusplus
}
#endif
#endif /* OEQ_B200_H */
