// "uvw" backward pass on the 5th-generation tensor cores (tcgen05, TMEM accumulators), FP32 in / FP32 out
// with 3xTF32 error compensation, for shared weights and second-input multiplicity 1.  Two kernels:
//
//   oeq_uvw_tc_dw_kernel    dW_p[u,w] = sum_{b,k} T_p[b,u,k] * dZ[b,o,w,k]          (K = batch x components)
//   oeq_uvw_tc_dxy_kernel   dT_p[b,u,k] = sum_w W_p[u,w] * dZ[b,o,w,k]              (K = output multiplicity)
//                           dX[b,u,i] += sum_{jk} C_ijk y_j dT_k,  dY[b,j] += sum_{u,i,k} C_ijk x_i dT_k
//
// with T_p[b,u,k] = sum_{ij} C_p[i,j,k] x[b,u,i] y[b,j] as in the forward pass.  Both are GEMMs whose
// operands do not exist in memory in the needed layout; producer warps build them as K-major,
// 128-byte-swizzled [rows x 32] tiles split into TF32 hi and lo parts, one thread issues the MMAs, and
// epilogue warps drain tensor memory.  hi.hi and hi.lo go out as one MMA over a B tile of 2 N rows
// (hi tile followed by lo tile), lo.hi as a second one, because issuing an MMA costs more than running it.
//
// Replaces the uvw branches of the reference's backward kernel and its warp-level matmul
// (openequivariance/templates/loop_unroll_tp.cuh:176-219, openequivariance/templates/wmm.cuh:1-88).
// Every wait is bounded; on expiry the role records a code in *status and stops, and the CTA still frees
// its tensor memory.
#pragma once
#include "oeq_common.cuh"
#include "tc_common.cuh"

namespace oeq {
using namespace oeqd;

struct UvwTcBwdParams {
    const float* X;
    const float* Y;
    const float* Wt;        // weights packed for the dX/dY kernel (oeq_uvw_pack_weights_t), else null
    const float* dZ;
    float* dX;
    float* dY;
    float* ws;              // [gridDim.x][W_NUMEL] partial weight gradients (dW kernel)
    long long batch;
    int* status;
};

constexpr int TB_PRODUCER_WARPS = 16;
constexpr int TB_EPILOGUE_WARPS = 4;
constexpr int TB_THREADS = (TB_PRODUCER_WARPS + 1 + TB_EPILOGUE_WARPS) * 32;
constexpr int TB_TILE = 128 * 128;             // one [128 rows x 32 tf32] swizzled tile
constexpr int ERR_TB_EMPTY = 31, ERR_TB_FULL = 32, ERR_TB_ACC_EMPTY = 33, ERR_TB_ACC_FULL = 34;

// Offset of W_p[u, w] (second-input multiplicity 1) in the kernel weight layout: 32-wide chunks, u-chunk major,
// each chunk stored [u][w] (reference: openequivariance/implementations/ComputationSchedule.py:146-230,427-471).
template <int P>
__device__ __forceinline__ int tb_weight_offset(int u, int w) {
    constexpr int MU = IN1_MUL[I_IN1[P]], MW = OUT_MUL[I_OUT[P]];
    if constexpr (MU <= 32 && MW <= 32) {
        return W_OFF[P] + u * MW + w;
    } else {
        const int uc = u >> 5, ul = u & 31, wc = w >> 5, wl = w & 31;
        const int ulen = (MU - (uc << 5)) < 32 ? (MU - (uc << 5)) : 32;
        const int wlen = (MW - (wc << 5)) < 32 ? (MW - (wc << 5)) : 32;
        return W_OFF[P] + (uc << 5) * MW + ulen * (wc << 5) + ul * wlen + wl;
    }
}

// rows of the batch owned by this CTA
__device__ __forceinline__ void tb_row_range(long long batch, long long& lo, long long& hi) {
    lo = batch * blockIdx.x / gridDim.x;
    hi = batch * (blockIdx.x + 1) / gridDim.x;
}

// ---- paths into an output irrep, grouped so that a group's first-input channels fill the 128 rows of an MMA
constexpr int tb_paths_into(int o) {
    int n = 0;
    for (int p = 0; p < N_INSTR; ++p) n += I_OUT[p] == o;
    return n;
}
constexpr int tb_nth_path(int o, int n) {      // n-th path into o, or -1
    for (int p = 0; p < N_INSTR; ++p)
        if (I_OUT[p] == o) {
            if (n == 0) return p;
            --n;
        }
    return -1;
}
constexpr int tb_slot(int o) {                 // rows per path inside a group: 64 if every path is that narrow
    for (int p = 0; p < N_INSTR; ++p)
        if (I_OUT[p] == o && IN1_MUL[I_IN1[p]] > 64) return 128;
    return 64;
}
constexpr int tb_per_group(int o) { return 128 / tb_slot(o); }
constexpr int tb_groups(int o) { return (tb_paths_into(o) + tb_per_group(o) - 1) / tb_per_group(o); }
constexpr int tb_mw_max() {
    int m = 16;
    for (int o = 0; o < N_OUT; ++o) m = OUT_MUL[o] > m ? OUT_MUL[o] : m;
    return m;
}
constexpr int TB_MW_MAX = tb_mw_max();

// =====================================================================================================
// dW kernel.  Per output irrep o and group of paths: D[(path,u), w] += sum over the CTA's batch rows.
// A stage holds RB = floor(32 / (2l+1)) batch rows: A = T^T as [128 (path,u) x 32 (row,k)], B = dZ^T as
// [MW w x 32 (row,k)], both hi and lo.  Every element of a stage is written (value or zero) each time.
// =====================================================================================================
constexpr int DW_B_HALF = TB_MW_MAX * 128;                       // [MW x 32] tile
constexpr int DW_STAGE_BYTES = 2 * TB_TILE + 2 * DW_B_HALF;      // A hi, A lo, B hi, B lo
constexpr int DW_STAGES = (200 * 1024) / DW_STAGE_BYTES < 4 ? (200 * 1024) / DW_STAGE_BYTES : 4;
constexpr int DW_ACC_COLS = 2 * TB_MW_MAX;                       // [hi.hi + lo.hi | hi.lo]
constexpr int DW_TMEM_COLS = 2 * DW_ACC_COLS <= 32 ? 32 : 2 * DW_ACC_COLS <= 64 ? 64 : 2 * DW_ACC_COLS <= 128 ? 128
                             : 2 * DW_ACC_COLS <= 256 ? 256 : 512;
constexpr int DW_OFF_BAR = DW_STAGES * DW_STAGE_BYTES;
constexpr int DW_SMEM_BYTES = DW_OFF_BAR + (2 * DW_STAGES + 4) * 8 + 16 + 1024;   // + alignment slack
static_assert(DW_STAGES >= 2, "two stages of the dW kernel must fit in shared memory");
static_assert(2 * TB_MW_MAX <= 256, "output multiplicity above 128");

struct DwBars {
    unsigned long long *full, *empty, *acc_full, *acc_empty;
    unsigned* tmem_slot;
    __device__ explicit DwBars(unsigned char* smem) {
        unsigned long long* b = reinterpret_cast<unsigned long long*>(smem + DW_OFF_BAR);
        full = b; empty = b + DW_STAGES; acc_full = b + 2 * DW_STAGES; acc_empty = acc_full + 2;
        tmem_slot = reinterpret_cast<unsigned*>(acc_empty + 2);
    }
};

template <int O, int GRP>
__device__ __forceinline__ bool dw_produce(const UvwTcBwdParams& p, unsigned char* smem, const DwBars& bars,
                                           long long row_lo, long long row_hi, long long& stage_it, int ptid) {
    constexpr int D3 = OUT_D[O], RB = 32 / D3, MW = OUT_MUL[O];
    constexpr int SLOT = tb_slot(O), PER = tb_per_group(O);
    constexpr int NPT = TB_PRODUCER_WARPS * 32;
    bool ok = true;
    for (long long b0 = row_lo; b0 < row_hi && ok; b0 += RB) {
        const int rows = (int)(row_hi - b0 < RB ? row_hi - b0 : RB);
        const int s = (int)(stage_it % DW_STAGES);
        const long long use = stage_it / DW_STAGES;
        if (use > 0) ok = mbar_wait(bars.empty + s, (unsigned)((use - 1) & 1), p.status, ERR_TB_EMPTY);
        if (!ok) break;
        unsigned char* a_hi = smem + s * DW_STAGE_BYTES;
        unsigned char* a_lo = a_hi + TB_TILE;
        unsigned char* b_hi = a_lo + TB_TILE;
        unsigned char* b_lo = b_hi + MW * 128;          // the lo tile follows the hi tile: one descriptor spans both
        // ---- A: T^T.  item = (row of the stage, slot row); a warp's 32 items share the path
        for (int item = ptid; item < RB * 128; item += NPT) {
            const int rr = item / 128, srow = item % 128;
            const int which = srow / SLOT, u = srow % SLOT;
            float t[D3];
#pragma unroll
            for (int k = 0; k < D3; ++k) t[k] = 0.f;
            sfor<0, PER>([&](auto j_) {
                constexpr int P = tb_nth_path(O, GRP * PER + j_);
                if constexpr (P >= 0) {
                    constexpr int a = I_IN1[P], b = I_IN2[P], D1 = IN1_D[a], D2 = IN2_D[b], MU = IN1_MUL[a];
                    if (which == j_ && u < MU && rr < rows) {
                        const float* xrow = p.X + (b0 + rr) * (long long)X_DIM + IN1_OFF[a] + u * D1;
                        const float* yrow = p.Y + (b0 + rr) * (long long)Y_DIM + IN2_OFF[b];
                        float x[D1], y[D2];
#pragma unroll
                        for (int i = 0; i < D1; ++i) x[i] = __ldg(xrow + i);
#pragma unroll
                        for (int j = 0; j < D2; ++j) y[j] = __ldg(yrow + j);
                        float xy = 0.f;
                        sfor<CG_BEGIN[P], CG_BEGIN[P + 1]>([&](auto n_) {
                            constexpr int N = n_;
                            if constexpr (N == CG_BEGIN[P] || CG_I[N] != CG_I[N - 1] || CG_J[N] != CG_J[N - 1])
                                xy = x[CG_I[N]] * y[CG_J[N]];
                            t[CG_K[N]] = fmaf(xy, (float)CG_V[N], t[CG_K[N]]);
                        });
                    }
                }
            });
#pragma unroll
            for (int k = 0; k < D3; ++k) {
                const int off = tc_swizzle(srow, rr * D3 + k);
                const float th = tf32_hi(t[k]);
                *reinterpret_cast<float*>(a_hi + off) = th;
                *reinterpret_cast<float*>(a_lo + off) = t[k] - th;
            }
        }
        // columns beyond RB * D3 are padding
        if constexpr (RB * D3 < 32) {
            for (int item = ptid; item < 128 * (32 - RB * D3); item += NPT) {
                const int srow = item % 128, col = RB * D3 + item / 128;
                const int off = tc_swizzle(srow, col);
                *reinterpret_cast<float*>(a_hi + off) = 0.f;
                *reinterpret_cast<float*>(a_lo + off) = 0.f;
            }
        }
        // ---- B: dZ^T.  consecutive threads read consecutive (w, k) of a batch row
        for (int item = ptid; item < 32 * MW; item += NPT) {
            int w, col;
            float g = 0.f;
            if (item < RB * MW * D3) {
                const int rr = item / (MW * D3), wk = item % (MW * D3);
                w = wk / D3;
                col = rr * D3 + wk % D3;
                if (rr < rows) g = __ldg(p.dZ + (b0 + rr) * (long long)Z_DIM + OUT_OFF[O] + wk);
            } else {                                    // padding columns
                const int e = item - RB * MW * D3;
                w = e % MW;
                col = RB * D3 + e / MW;
            }
            const int off = tc_swizzle(w, col);
            const float gh = tf32_hi(g);
            *reinterpret_cast<float*>(b_hi + off) = gh;
            *reinterpret_cast<float*>(b_lo + off) = g - gh;
        }
        fence_async_smem();
        __syncwarp();
        if ((ptid & 31) == 0) mbar_arrive(bars.full + s);
        ++stage_it;
    }
    return ok;
}

template <int O, int GRP>
__device__ __forceinline__ bool dw_mma(const UvwTcBwdParams& p, unsigned char* smem, const DwBars& bars, long long row_lo,
                                       long long row_hi, long long& stage_it, long long& acc_it, unsigned tmem_base) {
    constexpr int D3 = OUT_D[O], RB = 32 / D3, MW = OUT_MUL[O];
    constexpr unsigned IDESC = tc_instr_desc(MW), IDESC_WIDE = tc_instr_desc(2 * MW);
    if (row_lo >= row_hi) return true;
    const int t = (int)(acc_it & 1);
    const long long acc_use = acc_it >> 1;
    if (acc_use > 0 && !mbar_wait(bars.acc_empty + t, (unsigned)((acc_use - 1) & 1), p.status, ERR_TB_ACC_EMPTY)) return false;
    tc_fence_after();
    const unsigned tmem_d = tmem_base + (unsigned)(t * DW_ACC_COLS);
    const unsigned long long desc0 = tc_smem_desc(smem_u32(smem));
    unsigned accumulate = 0;
    for (long long b0 = row_lo; b0 < row_hi; b0 += RB) {
        const int s = (int)(stage_it % DW_STAGES);
        const long long use = stage_it / DW_STAGES;
        if (!mbar_wait(bars.full + s, (unsigned)(use & 1), p.status, ERR_TB_FULL)) return false;
        tc_fence_after();
        const unsigned long long da_hi = desc0 + (unsigned long long)((s * DW_STAGE_BYTES) >> 4);
        const unsigned long long da_lo = da_hi + (TB_TILE >> 4);
        const unsigned long long db = da_lo + (TB_TILE >> 4);        // hi tile, then lo tile
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
            tc_mma(tmem_d, da_hi + 2 * kk, db + 2 * kk, IDESC_WIDE, accumulate);   // [hi.hi | hi.lo]
            accumulate = 1;
            tc_mma(tmem_d, da_lo + 2 * kk, db + 2 * kk, IDESC, 1);                 // lo.hi into the first half
        }
        tc_commit(bars.empty + s);
        ++stage_it;
    }
    tc_commit(bars.acc_full + t);
    ++acc_it;
    return true;
}

template <int O, int GRP>
__device__ __forceinline__ bool dw_epilogue(const UvwTcBwdParams& p, const DwBars& bars, long long row_lo, long long row_hi,
                                            long long& acc_it, unsigned tmem_base, int ewarp, int lane) {
    constexpr int MW = OUT_MUL[O];
    constexpr int SLOT = tb_slot(O), PER = tb_per_group(O);
    float* out = p.ws + (long long)blockIdx.x * W_NUMEL;
    const int srow = ewarp * 32 + lane, which = srow / SLOT, u = srow % SLOT;
    if (row_lo >= row_hi) {   // no rows: this CTA's slice of the partial gradients is zero
        sfor<0, PER>([&](auto j_) {
            constexpr int P = tb_nth_path(O, GRP * PER + j_);
            if constexpr (P >= 0) {
                if (which == j_ && u < IN1_MUL[I_IN1[P]])
                    for (int w = 0; w < MW; ++w) out[tb_weight_offset<P>(u, w)] = 0.f;
            }
        });
        return true;
    }
    const int t = (int)(acc_it & 1);
    const long long use = acc_it >> 1;
    if (!mbar_wait(bars.acc_full + t, (unsigned)(use & 1), p.status, ERR_TB_ACC_FULL)) return false;
    tc_fence_after();
    // accumulator row = (path, u); a warp may only read the TMEM lanes of its own quarter
    const unsigned taddr = tmem_base + ((unsigned)(ewarp * 32) << 16) + (unsigned)(t * DW_ACC_COLS);
#pragma unroll
    for (int c0 = 0; c0 < MW; c0 += 16) {
        unsigned v[16], v2[16];
        tc_load16(taddr + (unsigned)c0, v);
        tc_load16(taddr + (unsigned)(MW + c0), v2);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        sfor<0, PER>([&](auto j_) {
            constexpr int P = tb_nth_path(O, GRP * PER + j_);
            if constexpr (P >= 0) {
                if (which == j_ && u < IN1_MUL[I_IN1[P]]) {
#pragma unroll
                    for (int c = 0; c < 16; ++c)
                        out[tb_weight_offset<P>(u, c0 + c)] = __uint_as_float(v[c]) + __uint_as_float(v2[c]);
                }
            }
        });
    }
    tc_fence_before();
    __syncwarp();
    if (lane == 0) mbar_arrive(bars.acc_empty + t);
    ++acc_it;
    return true;
}

__device__ void uvw_tc_dw(const UvwTcBwdParams& p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    const DwBars bars(smem);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    long long row_lo, row_hi;
    tb_row_range(p.batch, row_lo, row_hi);
    if (tid == 0) {
        for (int i = 0; i < DW_STAGES; ++i) {
            mbar_init(bars.full + i, TB_PRODUCER_WARPS);
            mbar_init(bars.empty + i, 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(bars.acc_full + i, 1);
            mbar_init(bars.acc_empty + i, TB_EPILOGUE_WARPS);
        }
        fence_mbar_init();
    }
    if (warp == TB_PRODUCER_WARPS) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(bars.tmem_slot)),
                     "n"(DW_TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem_base = *reinterpret_cast<volatile unsigned*>(bars.tmem_slot);

    if (warp < TB_PRODUCER_WARPS) {
        long long stage_it = 0;
        bool ok = true;
        sfor<0, N_OUT>([&](auto o_) {
            constexpr int O = o_;
            sfor<0, tb_groups(O)>([&](auto g_) {
                constexpr int GRP = g_;
                if (ok) ok = dw_produce<O, GRP>(p, smem, bars, row_lo, row_hi, stage_it, tid);
            });
        });
    } else if (warp == TB_PRODUCER_WARPS) {
        if (lane == 0) {
            long long stage_it = 0, acc_it = 0;
            bool ok = true;
            sfor<0, N_OUT>([&](auto o_) {
                constexpr int O = o_;
                sfor<0, tb_groups(O)>([&](auto g_) {
                    constexpr int GRP = g_;
                    if (ok) ok = dw_mma<O, GRP>(p, smem, bars, row_lo, row_hi, stage_it, acc_it, tmem_base);
                });
            });
        }
        __syncwarp();
    } else {
        long long acc_it = 0;
        bool ok = true;
        sfor<0, N_OUT>([&](auto o_) {
            constexpr int O = o_;
            sfor<0, tb_groups(O)>([&](auto g_) {
                constexpr int GRP = g_;
                if (ok) ok = dw_epilogue<O, GRP>(p, bars, row_lo, row_hi, acc_it, tmem_base, warp & 3, lane);
            });
        });
    }
    tc_fence_before();
    __syncthreads();
    if (warp == TB_PRODUCER_WARPS) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "n"(DW_TMEM_COLS) : "memory");
    }
}

}  // namespace oeq

#define OEQ_K_UVW_TC_DW 21

#if OEQ_KERNEL == OEQ_K_UVW_TC_DW
extern "C" __global__ void __launch_bounds__(oeq::TB_THREADS, 1) oeq_uvw_tc_dw_kernel(const oeq::UvwTcBwdParams p) {
    oeq::uvw_tc_dw(p);
}
#endif

// Fixed-order sum of the per-CTA partial weight gradients: dW[i] = sum_c ws[c][i].
extern "C" __global__ void oeq_reduce_partials(const float* ws, float* out, int n, long long groups) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float s = 0.f;
    for (long long g = 0; g < groups; ++g) s += ws[g * n + i];
    out[i] = s;
}
