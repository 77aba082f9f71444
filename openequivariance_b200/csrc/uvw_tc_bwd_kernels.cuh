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
    unsigned long long* prof;   // optional cycle accounting of CTA 0 (development aid), else null
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
        // the loads of dZ (the B operand, formed last) go out first: their latency overlaps the work on A
        constexpr int NBI = (32 * MW + NPT - 1) / NPT;
        float g[NBI];
#pragma unroll
        for (int q = 0; q < NBI; ++q) {
            const int item = ptid + q * NPT;
            g[q] = 0.f;
            if (item < RB * MW * D3) {
                const int rr = item / (MW * D3), wk = item % (MW * D3);
                if (rr < rows) g[q] = __ldg(p.dZ + (b0 + rr) * (long long)Z_DIM + OUT_OFF[O] + wk);
            }
        }
        // ---- A: T^T.  A thread keeps its slot row (path, u) and walks the stage's batch rows rr0, rr0 + 4, ...;
        // the global loads of a batch of rows go out together, so that their latency is paid once per batch
        {
            static_assert(NPT % 128 == 0, "a thread must keep its slot row");
            constexpr int STEP = NPT / 128, NI = (RB + STEP - 1) / STEP, NBATCH = NI < 4 ? NI : 4;
            const int srow = ptid % 128, which = srow / SLOT, u = srow % SLOT, rr0 = ptid / 128;
            bool done = false;
            sfor<0, PER>([&](auto j_) {
                constexpr int P = tb_nth_path(O, GRP * PER + j_);
                if constexpr (P >= 0) {
                    constexpr int a = I_IN1[P], b = I_IN2[P], D1 = IN1_D[a], D2 = IN2_D[b], MU = IN1_MUL[a];
                    if (which == j_ && u < MU) {
                        done = true;
                        for (int q0 = 0; q0 < NI; q0 += NBATCH) {
                            float x[NBATCH][D1], y[NBATCH][D2];
#pragma unroll
                            for (int q = 0; q < NBATCH; ++q) {
                                const int rr = rr0 + (q0 + q) * STEP;
                                const bool live = rr < rows;
                                const float* xrow = p.X + (b0 + (live ? rr : 0)) * (long long)X_DIM + IN1_OFF[a] + u * D1;
                                const float* yrow = p.Y + (b0 + (live ? rr : 0)) * (long long)Y_DIM + IN2_OFF[b];
#pragma unroll
                                for (int i = 0; i < D1; ++i) x[q][i] = live ? __ldg(xrow + i) : 0.f;
#pragma unroll
                                for (int j = 0; j < D2; ++j) y[q][j] = live ? __ldg(yrow + j) : 0.f;
                            }
#pragma unroll
                            for (int q = 0; q < NBATCH; ++q) {
                                const int rr = rr0 + (q0 + q) * STEP;
                                if (rr < RB) {
                                    float t[D3];
#pragma unroll
                                    for (int k = 0; k < D3; ++k) t[k] = 0.f;
                                    float xy = 0.f;
                                    sfor<CG_BEGIN[P], CG_BEGIN[P + 1]>([&](auto n_) {
                                        constexpr int N = n_;
                                        if constexpr (N == CG_BEGIN[P] || CG_I[N] != CG_I[N - 1] || CG_J[N] != CG_J[N - 1])
                                            xy = x[q][CG_I[N]] * y[q][CG_J[N]];
                                        t[CG_K[N]] = fmaf(xy, (float)CG_V[N], t[CG_K[N]]);
                                    });
#pragma unroll
                                    for (int k = 0; k < D3; ++k) {
                                        const int off = tc_swizzle(srow, rr * D3 + k);
                                        const float th = tf32_hi(t[k]);
                                        *reinterpret_cast<float*>(a_hi + off) = th;
                                        *reinterpret_cast<float*>(a_lo + off) = t[k] - th;
                                    }
                                }
                            }
                        }
                    }
                }
            });
            if (!done) {      // no path in this slot, or a channel beyond its multiplicity: zero rows
                for (int rr = rr0; rr < RB; rr += STEP)
#pragma unroll
                    for (int k = 0; k < D3; ++k) {
                        const int off = tc_swizzle(srow, rr * D3 + k);
                        *reinterpret_cast<float*>(a_hi + off) = 0.f;
                        *reinterpret_cast<float*>(a_lo + off) = 0.f;
                    }
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
        // ---- B: dZ^T.  consecutive threads hold consecutive (w, k) of a batch row (loaded above)
        {
#pragma unroll
            for (int q = 0; q < NBI; ++q) {
                const int item = ptid + q * NPT;
                if (item < 32 * MW) {
                    int w, col;
                    if (item < RB * MW * D3) {
                        const int rr = item / (MW * D3), wk = item % (MW * D3);
                        w = wk / D3;
                        col = rr * D3 + wk % D3;
                    } else {                                    // padding columns
                        const int e = item - RB * MW * D3;
                        w = e % MW;
                        col = RB * D3 + e / MW;
                    }
                    const int off = tc_swizzle(w, col);
                    const float gh = tf32_hi(g[q]);
                    *reinterpret_cast<float*>(b_hi + off) = gh;
                    *reinterpret_cast<float*>(b_lo + off) = g[q] - gh;
                }
            }
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

// =====================================================================================================
// dX / dY kernel.  Per output irrep o, chunk of RPC = floor(128 / (2l+1)) batch rows (A = dZ gathered once as
// [(row,k) x w] tiles) and path p into o (its weights W_p^T as the B operand, [u rows x w], hi tile followed
// by lo tile per 32-wide slice of w, double buffered in shared memory and fetched one path ahead):
// D[(row,k), u] = sum_w dZ[row,o,w,k] W_p[u,w] on the tensor cores.  The epilogue warps turn D (= dT) into dX and dY with the
// Clebsch-Gordan coefficients unrolled; dX and dY are cleared by the host and accumulated path by path by
// the CTA that owns the rows, in a fixed order.
// =====================================================================================================
constexpr int DX_PRODUCER_WARPS = 3;        // one fill per chunk serves all paths into the output irrep; 16 warps in
                                            // all leave 128 registers per thread for the epilogue's prefetch
constexpr int DX_EPILOGUE_WARPS = 12;       // the per-row arithmetic is what bounds the kernel
constexpr int DX_SUB = DX_EPILOGUE_WARPS / 4;   // epilogue warps per TMEM lane quarter
constexpr int DX_WARP_MMA = DX_PRODUCER_WARPS;
constexpr int DX_THREADS = (DX_PRODUCER_WARPS + 1 + DX_EPILOGUE_WARPS) * 32;
constexpr int ERR_DX_EMPTY = 41, ERR_DX_FULL = 42, ERR_DX_ACC_EMPTY = 43, ERR_DX_ACC_FULL = 44, ERR_DX_W = 45;

constexpr int dx_mup(int p) { return (IN1_MUL[I_IN1[p]] + 15) / 16 * 16; }          // rows of the weight tile
constexpr int dx_kblocks(int o) { return (OUT_MUL[o] + 31) / 32; }                   // 32-wide slices of w
constexpr int dx_wt_bytes(int p) { return dx_kblocks(I_OUT[p]) * 2 * dx_mup(p) * 128; }
constexpr int dx_wt_out_bytes(int o) {         // all paths into o
    int b = 0;
    for (int p = 0; p < N_INSTR; ++p)
        if (I_OUT[p] == o) b += dx_wt_bytes(p);
    return b;
}
constexpr int dx_wt_out_offset(int o) {        // byte offset of output o's block inside the packed transposed weights
    int b = 0;
    for (int q = 0; q < o; ++q) b += dx_wt_out_bytes(q);
    return b;
}
constexpr int dx_wt_local(int p_end) {         // byte offset of path p_end inside its output's block
    int b = 0;
    for (int p = 0; p < p_end; ++p)
        if (I_OUT[p] == I_OUT[p_end]) b += dx_wt_bytes(p);
    return b;
}
constexpr int dx_wt_offset(int p) { return dx_wt_out_offset(I_OUT[p]) + dx_wt_local(p); }
constexpr int dx_max(int (*f)(int), int n) {
    int m = 0;
    for (int i = 0; i < n; ++i) m = f(i) > m ? f(i) : m;
    return m;
}
constexpr int DX_KB_MAX = dx_max(dx_kblocks, N_OUT);
constexpr int DX_MUP_MAX = dx_max(dx_mup, N_INSTR);
constexpr int DX_WT_MAX = (dx_max(dx_wt_bytes, N_INSTR) + 1023) / 1024 * 1024;    // one path's tiles
constexpr int dx_row_floats(int p) { return IN1_MUL[I_IN1[p]] * IN1_D[I_IN1[p]]; }
constexpr int DX_ROWBUF = (dx_max(dx_row_floats, N_INSTR) * 4 + 15) / 16 * 16;       // one [channel][component] row
// Rows are walked in blocks of DX_BLOCK rows, each taken through all output irreps and paths before the next,
// so that a row's X, dX, dY and dZ values are still in cache when the next path needs them (every row is
// visited once per path).  The block is a whole number of chunks of the widest output irrep.
constexpr int dx_d3_max() {
    int m = 1;
    for (int o = 0; o < N_OUT; ++o)
        if (tb_paths_into(o) > 0 && OUT_D[o] > m) m = OUT_D[o];
    return m;
}
constexpr int DX_BLOCK = (128 / dx_d3_max()) * (128 / (128 / dx_d3_max()));
constexpr int DX_STAGE_BYTES = DX_KB_MAX * 2 * TB_TILE;         // per 32-wide slice of w: hi tile, lo tile
constexpr int DX_NA = 1;        // one set of A tiles: it serves all paths into the output irrep
constexpr int DX_ACC_COLS = 2 * DX_MUP_MAX;                      // [hi.hi + lo.hi | hi.lo]
constexpr int DX_NACC = 512 / DX_ACC_COLS < 4 ? 512 / DX_ACC_COLS : 4;
constexpr int DX_STG_PITCH = DX_MUP_MAX + 1;
constexpr int DX_OFF_A = 0;
constexpr int DX_OFF_W = DX_OFF_A + DX_NA * DX_STAGE_BYTES;
constexpr int DX_OFF_STG = DX_OFF_W + 2 * DX_WT_MAX;
constexpr int DX_OFF_ROW = DX_OFF_STG + (128 * DX_STG_PITCH * 4 + 15) / 16 * 16;
constexpr int DX_OFF_BAR = DX_OFF_ROW + DX_EPILOGUE_WARPS * 4 * DX_ROWBUF;   // per warp: two sets of an X row and a dX row
constexpr int DX_SMEM_BYTES = DX_OFF_BAR + (2 * DX_NA + 2 * DX_NACC + 4) * 8 + 16 + 1024;
static_assert(DX_ACC_COLS <= 256, "first-input multiplicity above 128");

struct DxBars {
    unsigned long long *full, *empty, *acc_full, *acc_empty, *w_full, *w_free;
    unsigned* tmem_slot;
    __device__ explicit DxBars(unsigned char* smem) {
        unsigned long long* b = reinterpret_cast<unsigned long long*>(smem + DX_OFF_BAR);
        full = b; empty = b + DX_NA; acc_full = b + 2 * DX_NA; acc_empty = acc_full + DX_NACC;
        w_full = acc_empty + DX_NACC; w_free = w_full + 2;       // one pair per weight buffer
        tmem_slot = reinterpret_cast<unsigned*>(w_free + 2);
    }
};

// A tiles of one chunk: element (row r * D3 + k, column w) = dZ[b0 + r, o, w, k]; every element is written
template <int O>
__device__ __forceinline__ bool dx_produce(const UvwTcBwdParams& p, unsigned char* smem, const DxBars& bars,
                                           long long row_lo, long long row_hi, long long& stage_it, int ptid) {
    constexpr int D3 = OUT_D[O], RPC = 128 / D3, MW = OUT_MUL[O], KB = dx_kblocks(O);
    constexpr int NPT = DX_PRODUCER_WARPS * 32;
    bool ok = true;
    for (long long b0 = row_lo; b0 < row_hi && ok; b0 += RPC) {
        const int rows = (int)(row_hi - b0 < RPC ? row_hi - b0 : RPC);
        const int s = (int)(stage_it % DX_NA);
        const long long use = stage_it / DX_NA;
        const bool prof = p.prof && blockIdx.x == 0 && ptid == 0;
        const long long t0 = prof ? clock64() : 0;
        if (use > 0) ok = mbar_wait(bars.empty + s, (unsigned)((use - 1) & 1), p.status, ERR_DX_EMPTY);
        const long long t1 = prof ? clock64() : 0;
        if (!ok) break;
        unsigned char* st = smem + DX_OFF_A + s * DX_STAGE_BYTES;
        // values: a thread keeps its (w, k) positions of a batch row and walks the rows, eight rows of loads
        // in flight at a time (consecutive threads read consecutive addresses)
        {
            constexpr int ROWLEN = MW * D3, NJ = (ROWLEN + NPT - 1) / NPT, RBATCH = 8;
            int kk_[NJ], tile_[NJ], chunk_[NJ], within_[NJ];
#pragma unroll
            for (int j = 0; j < NJ; ++j) {
                const int wk = ptid + j * NPT, w = wk / D3;
                kk_[j] = wk % D3;
                tile_[j] = (w >> 5) * 2 * TB_TILE;
                chunk_[j] = (w & 31) >> 2;
                within_[j] = (w & 3) << 2;
            }
            for (int r0 = 0; r0 < RPC; r0 += RBATCH) {
                float g[RBATCH][NJ];
#pragma unroll
                for (int rr = 0; rr < RBATCH; ++rr) {
                    const int r = r0 + rr;
                    const float* src = p.dZ + (b0 + r) * (long long)Z_DIM + OUT_OFF[O];
#pragma unroll
                    for (int j = 0; j < NJ; ++j) {
                        const int wk = ptid + j * NPT;
                        g[rr][j] = (r < rows && wk < ROWLEN) ? __ldg(src + wk) : 0.f;
                    }
                }
#pragma unroll
                for (int rr = 0; rr < RBATCH; ++rr) {
                    const int r = r0 + rr;
#pragma unroll
                    for (int j = 0; j < NJ; ++j) {
                        const int wk = ptid + j * NPT;
                        if (r < RPC && wk < ROWLEN) {
                            const int row = r * D3 + kk_[j];
                            const int off = (row >> 3) * 1024 + (row & 7) * 128 + (((chunk_[j] ^ (row & 7)) & 7) << 4) + within_[j];
                            unsigned char* hi = st + tile_[j];
                            const float gh = tf32_hi(g[rr][j]);
                            *reinterpret_cast<float*>(hi + off) = gh;
                            *reinterpret_cast<float*>(hi + TB_TILE + off) = g[rr][j] - gh;
                        }
                    }
                }
            }
        }
        // padding: rows beyond RPC * D3 and columns beyond MW
        constexpr int PAD_ROWS = 128 - RPC * D3, PAD_COLS = KB * 32 - MW;
        if constexpr (PAD_ROWS > 0) {
            for (int item = ptid; item < PAD_ROWS * KB * 32; item += NPT) {
                const int row = RPC * D3 + item / (KB * 32), col = item % (KB * 32);
                unsigned char* hi = st + (col >> 5) * 2 * TB_TILE;
                const int off = tc_swizzle(row, col & 31);
                *reinterpret_cast<float*>(hi + off) = 0.f;
                *reinterpret_cast<float*>(hi + TB_TILE + off) = 0.f;
            }
        }
        if constexpr (PAD_COLS > 0) {
            for (int item = ptid; item < RPC * D3 * PAD_COLS; item += NPT) {
                const int row = item / PAD_COLS, col = MW + item % PAD_COLS;
                unsigned char* hi = st + (col >> 5) * 2 * TB_TILE;
                const int off = tc_swizzle(row, col & 31);
                *reinterpret_cast<float*>(hi + off) = 0.f;
                *reinterpret_cast<float*>(hi + TB_TILE + off) = 0.f;
            }
        }
        fence_async_smem();
        __syncwarp();
        if ((ptid & 31) == 0) mbar_arrive(bars.full + s);
        if (prof) {
            atomicAdd(p.prof + 0, (unsigned long long)(t1 - t0));
            atomicAdd(p.prof + 1, (unsigned long long)(clock64() - t1));
            atomicAdd(p.prof + 2, 1ull);
        }
        ++stage_it;
    }
    return ok;
}

constexpr int dx_next_path(int p) {            // next path into the same output irrep, cyclically
    for (int q = p + 1; q < N_INSTR; ++q)
        if (I_OUT[q] == I_OUT[p]) return q;
    for (int q = 0; q < p; ++q)
        if (I_OUT[q] == I_OUT[p]) return q;
    return p;
}
constexpr int dx_last_path(int o) {
    int last = -1;
    for (int p = 0; p < N_INSTR; ++p)
        if (I_OUT[p] == o) last = p;
    return last;
}

// Start the copy of path P's weight tiles into weight buffer `buf` (after the MMAs that read its previous
// contents are done).  w_cnt[buf] counts the copies into that buffer.
template <int P>
__device__ __forceinline__ bool dx_load_w(const UvwTcBwdParams& p, unsigned char* smem, const DxBars& bars, int buf,
                                          long long (&w_cnt)[2]) {
    const long long k = w_cnt[buf];
    if (k > 0 && !mbar_wait(bars.w_free + buf, (unsigned)((k - 1) & 1), p.status, ERR_DX_W)) return false;
    constexpr int TOTAL = dx_wt_bytes(P);
    mbar_arrive_expect_tx(bars.w_full + buf, (unsigned)TOTAL);
    const unsigned char* src = reinterpret_cast<const unsigned char*>(p.Wt) + dx_wt_offset(P);
    for (int off = 0; off < TOTAL; off += 32768) {
        const int n = TOTAL - off < 32768 ? TOTAL - off : 32768;
        bulk_g2s(smem + DX_OFF_W + buf * DX_WT_MAX + off, src + off, (unsigned)n, bars.w_full + buf);
    }
    ++w_cnt[buf];
    return true;
}

template <int O>
__device__ __forceinline__ bool dx_mma(const UvwTcBwdParams& p, unsigned char* smem, const DxBars& bars, long long row_lo,
                                       long long row_hi, long long& stage_it, long long& acc_it, long long (&w_cnt)[2],
                                       unsigned tmem_base) {
    constexpr int D3 = OUT_D[O], RPC = 128 / D3, KB = dx_kblocks(O);
    if (row_lo >= row_hi) return true;
    const unsigned long long a_desc0 = tc_smem_desc(smem_u32(smem + DX_OFF_A));
    const unsigned long long w_desc0 = tc_smem_desc(smem_u32(smem + DX_OFF_W));
    bool ok = true;
    bool fetched = false;      // the weights of the coming unit are already on their way
    for (long long b0 = row_lo; b0 < row_hi && ok; b0 += RPC) {
        const int s = (int)(stage_it % DX_NA);
        const long long use = stage_it / DX_NA;
        const bool prof = p.prof && blockIdx.x == 0;
        const long long t1 = prof ? clock64() : 0;
        if (!mbar_wait(bars.full + s, (unsigned)(use & 1), p.status, ERR_DX_FULL)) return false;
        const long long t2 = prof ? clock64() : 0;
        tc_fence_after();
        const bool last_chunk = b0 + RPC >= row_hi;
        sfor<0, N_INSTR>([&](auto p_) {
            constexpr int P = p_;
            if constexpr (I_OUT[P] == O) {
                constexpr int MUP = dx_mup(P);
                constexpr unsigned IDESC = tc_instr_desc(MUP), IDESC_WIDE = tc_instr_desc(2 * MUP);
                if (ok) {
                    const int wb = (int)(acc_it & 1);          // weight buffer of this unit
                    if (!fetched) ok = dx_load_w<P>(p, smem, bars, wb, w_cnt);
                    // the next unit's weights travel while this unit's MMAs run
                    fetched = !(last_chunk && P == dx_last_path(O));
                    if (ok && fetched) ok = dx_load_w<dx_next_path(P)>(p, smem, bars, wb ^ 1, w_cnt);
                    const int t = (int)(acc_it % DX_NACC);
                    const long long acc_use = acc_it / DX_NACC;
                    const long long t0 = prof ? clock64() : 0;
                    if (ok && acc_use > 0) ok = mbar_wait(bars.acc_empty + t, (unsigned)((acc_use - 1) & 1), p.status, ERR_DX_ACC_EMPTY);
                    if (ok) ok = mbar_wait(bars.w_full + wb, (unsigned)((w_cnt[wb] - 1) & 1), p.status, ERR_DX_W);
                    if (prof) atomicAdd(p.prof + 8, (unsigned long long)(clock64() - t0));
                    if (ok) {
                        tc_fence_after();
                        const unsigned tmem_d = tmem_base + (unsigned)(t * DX_ACC_COLS);
                        unsigned accumulate = 0;
#pragma unroll
                        for (int kb = 0; kb < KB; ++kb) {
                            const unsigned long long da_hi = a_desc0 + (unsigned long long)((s * DX_STAGE_BYTES + kb * 2 * TB_TILE) >> 4);
                            const unsigned long long da_lo = da_hi + (TB_TILE >> 4);
                            // this path's tiles of the slice: hi rows, then lo rows
                            const unsigned long long db = w_desc0 + (unsigned long long)((wb * DX_WT_MAX + kb * 2 * MUP * 128) >> 4);
#pragma unroll
                            for (int kk = 0; kk < 4; ++kk) {
                                tc_mma(tmem_d, da_hi + 2 * kk, db + 2 * kk, IDESC_WIDE, accumulate);   // [hi.hi | hi.lo]
                                accumulate = 1;
                                tc_mma(tmem_d, da_lo + 2 * kk, db + 2 * kk, IDESC, 1);                 // lo.hi into the first half
                            }
                        }
                        tc_commit(bars.w_free + wb);
                        tc_commit(bars.acc_full + t);
                        ++acc_it;
                    }
                }
            }
        });
        if (!ok) return false;
        tc_commit(bars.empty + s);        // the A tiles may be refilled once the MMAs of all paths have read them
        if (prof) {
            atomicAdd(p.prof + 9, (unsigned long long)(t2 - t1));
            atomicAdd(p.prof + 10, (unsigned long long)(clock64() - t2));
        }
        ++stage_it;
    }
    return ok;
}

// AND-reduction of a flag over the epilogue warps (hardware barrier 1).
__device__ __forceinline__ bool dx_epilogue_all(bool ok) {
    unsigned r;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\tsetp.ne.b32 q, %1, 0;\n\t"
        "bar.red.and.pred p, 1, %2, q;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(r)
        : "r"((unsigned)ok), "n"(DX_EPILOGUE_WARPS * 32)
        : "memory");
    return r != 0;
}

// One (chunk, path) unit: accumulator -> staging buffer -> dX, dY of the chunk's rows.
template <int P>
__device__ __forceinline__ bool dx_epilogue_unit(const UvwTcBwdParams& p, unsigned char* smem, const DxBars& bars,
                                                 long long b0, int rows, long long& acc_it, unsigned tmem_base,
                                                 int ewarp, int lane) {
    constexpr int O = I_OUT[P], a = I_IN1[P], b = I_IN2[P];
    constexpr int D1 = IN1_D[a], D2 = IN2_D[b], D3 = OUT_D[O], RPC = 128 / D3, MU = IN1_MUL[a], MUP = dx_mup(P);
    float* stg = reinterpret_cast<float*>(smem + DX_OFF_STG);
    // a warp may only read the TMEM lanes of its own quarter, 32 * (warp index in the CTA mod 4); the
    // warps of a quarter split the columns in slices of 16
    const int quarter = (DX_WARP_MMA + 1 + ewarp) & 3, sub = ewarp >> 2;
    bool ok = true;
    {
        const int t = (int)(acc_it % DX_NACC);
        const long long use = acc_it / DX_NACC;
        const bool prof = p.prof && blockIdx.x == 0 && ewarp == 0 && lane == 0;
        const long long t0 = prof ? clock64() : 0;
        ok = mbar_wait(bars.acc_full + t, (unsigned)(use & 1), p.status, ERR_DX_ACC_FULL);
        ok = dx_epilogue_all(ok);          // the warps must agree before anyone touches the staging buffer
        const long long t1 = prof ? clock64() : 0;
        if (!ok) return false;
        tc_fence_after();
        // accumulator row m = 32 * quarter + lane holds (row m / D3, component m % D3) for all u
        const unsigned taddr = tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)(t * DX_ACC_COLS);
#pragma unroll
        for (int c16 = 0; c16 < MUP / 16; ++c16) {
            if (c16 % DX_SUB == sub) {
                const int c = 16 * c16;
                unsigned v[16], v2[16];
                tc_load16(taddr + (unsigned)c, v);
                tc_load16(taddr + (unsigned)(MUP + c), v2);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int q = 0; q < 16; ++q)
                    stg[(quarter * 32 + lane) * DX_STG_PITCH + c + q] = __uint_as_float(v[q]) + __uint_as_float(v2[q]);
            }
        }
        tc_fence_before();
        asm volatile("bar.sync 1, %0;" ::"n"(DX_EPILOGUE_WARPS * 32) : "memory");
        if (ewarp == 0 && lane == 0) mbar_arrive(bars.acc_empty + t);   // the accumulator tile may be overwritten
        const long long t2 = prof ? clock64() : 0;
        // One warp per batch row, lanes over the channels: dX by the owning lane, dY reduced over the warp.
        // X and dX rows are [channel][component]: they travel as contiguous floats (lane = flat index) between
        // global memory and the warp's own shared-memory row buffers, because a lane-per-channel access would
        // touch 2l+1 times the sectors it uses.  The rows of the warp's next batch row are copied asynchronously
        // (cp.async into the other buffer set) while the current row is computed.
        {
            constexpr int NU = (MU + 31) / 32, ROW = MU * D1, NF = (ROW + 31) / 32;
            static_assert(NU <= 4, "first-input multiplicity above 128");
            unsigned char* rowbase = smem + DX_OFF_ROW + ewarp * 4 * DX_ROWBUF;
            auto xbuf = [&](int set) { return reinterpret_cast<float*>(rowbase + set * 2 * DX_ROWBUF); };
            auto dbuf = [&](int set) { return reinterpret_cast<float*>(rowbase + set * 2 * DX_ROWBUF + DX_ROWBUF); };
            auto prefetch = [&](int r, int set) {
                const float* xrow = p.X + (b0 + r) * (long long)X_DIM + IN1_OFF[a];
                const float* dxrow = p.dX + (b0 + r) * (long long)X_DIM + IN1_OFF[a];
#pragma unroll
                for (int q = 0; q < NF; ++q) {
                    const int idx = lane + 32 * q;
                    if (idx < ROW) {
                        cp_async_elem<4>(xbuf(set) + idx, xrow + idx);
                        cp_async_elem<4>(dbuf(set) + idx, dxrow + idx);
                    }
                }
                asm volatile("cp.async.commit_group;" ::: "memory");
            };
            auto load_y = [&](int r, float (&y)[D2], float (&oy)[D2]) {
                const float* yrow = p.Y + (b0 + r) * (long long)Y_DIM + IN2_OFF[b];
                const float* dyrow = p.dY + (b0 + r) * (long long)Y_DIM + IN2_OFF[b];
#pragma unroll
                for (int j = 0; j < D2; ++j) {
                    y[j] = __ldg(yrow + j);
                    oy[j] = lane == 0 ? dyrow[j] : 0.f;
                }
            };
            float yA[D2], oyA[D2];
            int set = 0;
            if (ewarp < rows) {
                prefetch(ewarp, 0);
                load_y(ewarp, yA, oyA);
            }
            for (int r = ewarp; r < rows; r += DX_EPILOGUE_WARPS) {
                float yB[D2], oyB[D2];
                const int rn = r + DX_EPILOGUE_WARPS;
                if (rn < rows) {
                    prefetch(rn, set ^ 1);
                    load_y(rn, yB, oyB);
                    asm volatile("cp.async.wait_group 1;" ::: "memory");
                } else {
                    asm volatile("cp.async.wait_group 0;" ::: "memory");
                }
                __syncwarp();
                const long long tr0 = prof ? clock64() : 0;
                float* xs = xbuf(set);
                float* ds = dbuf(set);
                float dy[D2];
#pragma unroll
                for (int j = 0; j < D2; ++j) dy[j] = 0.f;
#pragma unroll
                for (int v = 0; v < NU; ++v) {
                    const int u = lane + 32 * v;
                    if (u < MU) {
                        float x[D1], old[D1], g[D3];
#pragma unroll
                        for (int i = 0; i < D1; ++i) {
                            x[i] = xs[u * D1 + i];
                            old[i] = ds[u * D1 + i];
                        }
#pragma unroll
                        for (int k = 0; k < D3; ++k) g[k] = stg[(r * D3 + k) * DX_STG_PITCH + u];
                        sfor<CG_BEGIN[P], CG_BEGIN[P + 1]>([&](auto n_) {
                            constexpr int N = n_;
                            const float cg = (float)CG_V[N] * g[CG_K[N]];
                            old[CG_I[N]] = fmaf(cg, yA[CG_J[N]], old[CG_I[N]]);
                            dy[CG_J[N]] = fmaf(cg, x[CG_I[N]], dy[CG_J[N]]);
                        });
#pragma unroll
                        for (int i = 0; i < D1; ++i) ds[u * D1 + i] = old[i];    // a lane rewrites only what it read
                    }
                }
                __syncwarp();
                float* dxrow = p.dX + (b0 + r) * (long long)X_DIM + IN1_OFF[a];
#pragma unroll
                for (int q = 0; q < NF; ++q)
                    if (lane + 32 * q < ROW) dxrow[lane + 32 * q] = ds[lane + 32 * q];
                __syncwarp();          // the buffer set is refilled two rows later
                const long long tr1 = prof ? clock64() : 0;
#pragma unroll
                for (int j = 0; j < D2; ++j) {
                    float sum = dy[j];
#pragma unroll
                    for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
                    if (lane == 0) p.dY[(b0 + r) * (long long)Y_DIM + IN2_OFF[b] + j] = oyA[j] + sum;
                }
                if (prof) {
                    atomicAdd(p.prof + 24, (unsigned long long)(tr1 - tr0));          // compute + dX stores
                    atomicAdd(p.prof + 25, (unsigned long long)(clock64() - tr1));    // dY reduction + stores
                    atomicAdd(p.prof + 26, 1ull);
                }
                if (rn < rows) {
#pragma unroll
                    for (int j = 0; j < D2; ++j) { yA[j] = yB[j]; oyA[j] = oyB[j]; }
                }
                set ^= 1;
            }
        }
        // the staging buffer is rewritten by the next tile, and the next path adds to the same dX / dY rows
        const long long t3 = prof ? clock64() : 0;
        __threadfence_block();
        asm volatile("bar.sync 1, %0;" ::"n"(DX_EPILOGUE_WARPS * 32) : "memory");
        if (prof) {
            atomicAdd(p.prof + 16, (unsigned long long)(t1 - t0));
            atomicAdd(p.prof + 17, (unsigned long long)(t2 - t1));
            atomicAdd(p.prof + 18, (unsigned long long)(t3 - t2));
            atomicAdd(p.prof + 19, (unsigned long long)(clock64() - t3));
        }
        ++acc_it;
    }
    return ok;
}

template <int O>
__device__ __forceinline__ bool dx_epilogue(const UvwTcBwdParams& p, unsigned char* smem, const DxBars& bars,
                                            long long row_lo, long long row_hi, long long& acc_it, unsigned tmem_base,
                                            int ewarp, int lane) {
    constexpr int RPC = 128 / OUT_D[O];
    bool ok = true;
    for (long long b0 = row_lo; b0 < row_hi && ok; b0 += RPC) {
        const int rows = (int)(row_hi - b0 < RPC ? row_hi - b0 : RPC);
        sfor<0, N_INSTR>([&](auto p_) {
            constexpr int P = p_;
            if constexpr (I_OUT[P] == O) {
                if (ok) ok = dx_epilogue_unit<P>(p, smem, bars, b0, rows, acc_it, tmem_base, ewarp, lane);
            }
        });
    }
    return ok;
}

__device__ void uvw_tc_dxy(const UvwTcBwdParams& p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    const DxBars bars(smem);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    long long row_lo, row_hi;
    tb_row_range(p.batch, row_lo, row_hi);
    if (tid == 0) {
        for (int i = 0; i < DX_NA; ++i) {
            mbar_init(bars.full + i, DX_PRODUCER_WARPS);
            mbar_init(bars.empty + i, 1);
        }
        for (int i = 0; i < DX_NACC; ++i) {
            mbar_init(bars.acc_full + i, 1);
            mbar_init(bars.acc_empty + i, 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(bars.w_full + i, 1);
            mbar_init(bars.w_free + i, 1);
        }
        fence_mbar_init();
    }
    if (warp == DX_WARP_MMA) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(bars.tmem_slot)),
                     "n"(512)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem_base = *reinterpret_cast<volatile unsigned*>(bars.tmem_slot);

    if (warp < DX_PRODUCER_WARPS) {
        long long stage_it = 0;
        bool ok = true;
        for (long long blk = row_lo; blk < row_hi && ok; blk += DX_BLOCK) {
            const long long blk_hi = blk + DX_BLOCK < row_hi ? blk + DX_BLOCK : row_hi;
            sfor<0, N_OUT>([&](auto o_) {
                constexpr int O = o_;
                if constexpr (tb_paths_into(O) > 0) {
                    if (ok) ok = dx_produce<O>(p, smem, bars, blk, blk_hi, stage_it, tid);
                }
            });
        }
    } else if (warp == DX_WARP_MMA) {
        if (lane == 0) {
            long long stage_it = 0, acc_it = 0;
            long long w_cnt[2] = {0, 0};
            bool ok = true;
            for (long long blk = row_lo; blk < row_hi && ok; blk += DX_BLOCK) {
                const long long blk_hi = blk + DX_BLOCK < row_hi ? blk + DX_BLOCK : row_hi;
                sfor<0, N_OUT>([&](auto o_) {
                    constexpr int O = o_;
                    if constexpr (tb_paths_into(O) > 0) {
                        if (ok) ok = dx_mma<O>(p, smem, bars, blk, blk_hi, stage_it, acc_it, w_cnt, tmem_base);
                    }
                });
            }
        }
        __syncwarp();
    } else {
        long long acc_it = 0;
        bool ok = true;
        for (long long blk = row_lo; blk < row_hi && ok; blk += DX_BLOCK) {
            const long long blk_hi = blk + DX_BLOCK < row_hi ? blk + DX_BLOCK : row_hi;
            sfor<0, N_OUT>([&](auto o_) {
                constexpr int O = o_;
                if constexpr (tb_paths_into(O) > 0) {
                    if (ok) ok = dx_epilogue<O>(p, smem, bars, blk, blk_hi, acc_it, tmem_base, warp - DX_WARP_MMA - 1, lane);
                }
            });
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == DX_WARP_MMA) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "n"(512) : "memory");
    }
}

}  // namespace oeq

#define OEQ_K_UVW_TC_DW 21
#define OEQ_K_UVW_TC_DXY 22

#if OEQ_KERNEL == OEQ_K_UVW_TC_DW
extern "C" __global__ void __launch_bounds__(oeq::TB_THREADS, 1) oeq_uvw_tc_dw_kernel(const oeq::UvwTcBwdParams p) {
    oeq::uvw_tc_dw(p);
}
#elif OEQ_KERNEL == OEQ_K_UVW_TC_DXY
extern "C" __global__ void __launch_bounds__(oeq::DX_THREADS, 1) oeq_uvw_tc_dxy_kernel(const oeq::UvwTcBwdParams p) {
    oeq::uvw_tc_dxy(p);
}

// Splits the shared weights into TF32 hi / lo parts, transposed for the dX/dY kernel: per path and per
// 32-wide slice of w a [u rows x 32] K-major tile with the 128-byte swizzle for hi, followed by one for lo.
// Rows of u beyond the multiplicity (up to a multiple of 16) and columns of w beyond the output multiplicity are zero.
extern "C" __global__ void oeq_uvw_pack_weights_t(const float* __restrict__ W, float* __restrict__ packed) {
    using namespace oeqd;
    const int tid = blockIdx.x * blockDim.x + threadIdx.x, nthreads = gridDim.x * blockDim.x;
    oeq::sfor<0, N_INSTR>([&](auto p_) {
        constexpr int P = p_;
        constexpr int O = I_OUT[P], MU = IN1_MUL[I_IN1[P]], MW = OUT_MUL[O];
        constexpr int KB = oeq::dx_kblocks(O), MUP = oeq::dx_mup(P);
        unsigned char* base = reinterpret_cast<unsigned char*>(packed) + oeq::dx_wt_offset(P);
        for (int e = tid; e < KB * MUP * 32; e += nthreads) {
            const int col = e & 31, u = (e >> 5) % MUP, kb = e / (32 * MUP);
            const int w = kb * 32 + col;
            const float v = (u < MU && w < MW) ? W[oeq::tb_weight_offset<P>(u, w)] : 0.f;
            const float hi = oeq::tf32_round(v), lo = oeq::tf32_round(v - hi);
            unsigned char* blk = base + kb * 2 * MUP * 128;
            *reinterpret_cast<float*>(blk + oeq::tc_swizzle(u, col)) = hi;
            *reinterpret_cast<float*>(blk + MUP * 128 + oeq::tc_swizzle(u, col)) = lo;
        }
    });
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
