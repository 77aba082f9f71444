// "uvw" forward pass on the 5th-generation tensor cores (tcgen05, TMEM accumulators), FP32 in / FP32
// out with 3xTF32 error compensation, for shared weights and second-input multiplicity 1.
//
//   Z[b,o,w,k] = sum_{paths p -> o} sum_u W_p[u,w] * T_p[b,u,k],   T_p[b,u,k] = sum_{ij} C_p[i,j,k] x[b,u,i] y[b,j]
//
// is a GEMM whose A operand does not exist in memory: rows are (batch row, k), the K axis is (path, u),
// N is the output multiplicity.  Per output irrep o the CTA keeps W (split into TF32 "hi" and "lo"
// parts, pre-swizzled by oeq_uvw_pack_weights) resident in shared memory and walks its share of the
// batch in chunks of floor(128 / (2l+1)) rows:
//
//   * 16 producer warps form T with the Clebsch-Gordan constants unrolled, split every value into
//     hi = tf32(t), lo = tf32(t - hi), and store both as K-major 128-byte-swizzled [128 x 32] tiles;
//   * one thread issues tcgen05.mma (M = 128, N = mul_out, K = 8 per instruction) three times per K step
//     (hi.hi + hi.lo + lo.hi) into a ring of TMEM accumulator tiles, and hands shared-memory stages
//     and accumulators on with tcgen05.commit -> mbarrier;
//   * 4 epilogue warps read accumulators with tcgen05.ld, transpose (row,k)-major tiles through a
//     padded shared-memory buffer and write Z rows coalesced.
//
// Replaces the reference's per-row warp matmul (openequivariance/templates/wmm.cuh:1-88,
// openequivariance/templates/loop_unroll_tp.cuh:54-83).  Every wait is bounded; on expiry the role
// records a code in *status and stops, and the CTA still frees its tensor memory.
#pragma once
#include "oeq_common.cuh"
#include "tc_common.cuh"

namespace oeq {
using namespace oeqd;

struct UvwTcParams {
    const float* X;
    const float* Y;
    const float* Wpacked;   // output of oeq_uvw_pack_weights
    float* Z;
    long long batch;
    int* status;
    unsigned long long* prof;   // optional cycle accounting of CTA 0 (development aid), else null
};

constexpr int TC_PRODUCER_WARPS = 16;
constexpr int TC_EPILOGUE_WARPS = 4;
constexpr int TC_THREADS = (TC_PRODUCER_WARPS + 1 + TC_EPILOGUE_WARPS) * 32;
constexpr int TC_NA = 2;                       // A-operand stages
constexpr int TC_STAGE_HALF = 128 * 128;       // one [128 rows x 32 tf32] swizzled tile
constexpr int TC_STAGE_BYTES = 2 * TC_STAGE_HALF;   // hi + lo
constexpr int ERR_TC_A_EMPTY = 11, ERR_TC_A_FULL = 12, ERR_TC_ACC_EMPTY = 13, ERR_TC_ACC_FULL = 14, ERR_TC_W = 15;

// ---- compile-time geometry ------------------------------------------------------------------
constexpr int tc_khalves(int p) { return (IN1_MUL[I_IN1[p]] + 31) / 32; }
constexpr int tc_blocks_before(int o, int p_end) {   // [MW x 32] weight blocks of output o before path p_end
    int n = 0;
    for (int p = 0; p < p_end; ++p)
        if (I_OUT[p] == o) n += tc_khalves(p);
    return n;
}
constexpr int tc_block_bytes(int o) { return OUT_MUL[o] * 128; }                 // one hi (or lo) block
constexpr int tc_w_bytes(int o) { return tc_blocks_before(o, N_INSTR) * 2 * tc_block_bytes(o); }
constexpr int tc_w_offset(int o) {   // byte offset of output o inside the packed weight buffer
    int b = 0;
    for (int q = 0; q < o; ++q) b += tc_w_bytes(q);
    return b;
}
constexpr int tc_w_max() {
    int m = 0;
    for (int o = 0; o < N_OUT; ++o) m = tc_w_bytes(o) > m ? tc_w_bytes(o) : m;
    return m;
}
constexpr int tc_mw_max() {
    int m = 16;
    for (int o = 0; o < N_OUT; ++o) m = OUT_MUL[o] > m ? OUT_MUL[o] : m;
    return m;
}
constexpr bool tc_wide(int o) { return 2 * OUT_MUL[o] <= 256; }
constexpr int tc_acc_cols(int o) { return tc_wide(o) ? 2 * OUT_MUL[o] : OUT_MUL[o]; }
// One ring of accumulator tiles serves all output irreps: equal tile width and count for all of them, so that
// tile index and barrier phase follow from one running counter.
constexpr int tc_acc_cols_max() {
    int m = 16;
    for (int o = 0; o < N_OUT; ++o) m = tc_acc_cols(o) > m ? tc_acc_cols(o) : m;
    return m;
}
constexpr int TC_ACC_COLS = tc_acc_cols_max();
constexpr int TC_W_MAX = tc_w_max();
constexpr int TC_MW_MAX = tc_mw_max();
constexpr int TC_STG_PITCH = TC_MW_MAX + 1;    // floats per staged accumulator row (odd: conflict free)
constexpr int TC_TMEM_COLS = 512;

// shared memory map (1024-byte aligned base): [A stages][W of one output][epilogue staging][barriers]
constexpr int TC_OFF_A = 0;
constexpr int TC_OFF_W = TC_OFF_A + TC_NA * TC_STAGE_BYTES;
constexpr int TC_OFF_STG = TC_OFF_W + (TC_W_MAX + 1023) / 1024 * 1024;
constexpr int TC_OFF_BAR = TC_OFF_STG + (128 * TC_STG_PITCH * 4 + 15) / 16 * 16;
constexpr int TC_MAX_ACC = 32;
constexpr int TC_NACC = TC_TMEM_COLS / TC_ACC_COLS < TC_MAX_ACC ? TC_TMEM_COLS / TC_ACC_COLS : TC_MAX_ACC;
constexpr int TC_SMEM_BYTES = TC_OFF_BAR + (2 * TC_NA + 2 * TC_MAX_ACC + 2) * 8 + 16 + 1024;   // + alignment slack

struct TcBars {
    unsigned long long* a_full;     // [TC_NA]
    unsigned long long* a_empty;    // [TC_NA]
    unsigned long long* acc_full;   // [TC_MAX_ACC]
    unsigned long long* acc_empty;  // [TC_MAX_ACC]
    unsigned long long* w_full;
    unsigned long long* w_free;
    unsigned* tmem_slot;
    __device__ explicit TcBars(unsigned char* base) {
        unsigned long long* b = reinterpret_cast<unsigned long long*>(base + TC_OFF_BAR);
        a_full = b; a_empty = b + TC_NA; acc_full = b + 2 * TC_NA; acc_empty = acc_full + TC_MAX_ACC;
        w_full = acc_empty + TC_MAX_ACC; w_free = w_full + 1;
        tmem_slot = reinterpret_cast<unsigned*>(w_free + 1);
    }
};

// rows of the batch owned by this CTA
__device__ __forceinline__ void tc_row_range(long long batch, long long& lo, long long& hi) {
    lo = batch * blockIdx.x / gridDim.x;
    hi = batch * (blockIdx.x + 1) / gridDim.x;
}

// ---------------------------------------------------------------------------- producers
template <int O>
__device__ __forceinline__ bool tc_produce_output(const UvwTcParams& p, unsigned char* smem, const TcBars& bars,
                                                  long long row_lo, long long row_hi, long long& stage_it, int warp,
                                                  int lane) {
    constexpr int D3 = OUT_D[O];
    constexpr int RPC = 128 / D3;
    bool ok = true;
    for (long long b0 = row_lo; b0 < row_hi && ok; b0 += RPC) {
        const int rows = (int)(row_hi - b0 < RPC ? row_hi - b0 : RPC);
        sfor<0, N_INSTR>([&](auto p_) {
            constexpr int P = p_;
            if constexpr (I_OUT[P] == O) {
                constexpr int a = I_IN1[P], b = I_IN2[P];
                constexpr int D1 = IN1_D[a], D2 = IN2_D[b], MU = IN1_MUL[a];
                for (int h = 0; h < tc_khalves(P) && ok; ++h) {
                    const int s = (int)(stage_it % TC_NA);
                    const long long use = stage_it / TC_NA;
                    // all global loads of this warp's rows go out first, so their latency is paid once per
                    // stage and overlaps the wait for the stage to be handed back
                    constexpr int RW = (RPC + TC_PRODUCER_WARPS - 1) / TC_PRODUCER_WARPS;
                    const int u = h * 32 + lane;
                    float xs[RW][D1], ys[RW][D2];
#pragma unroll
                    for (int q = 0; q < RW; ++q) {
                        const int r = warp + q * TC_PRODUCER_WARPS;
                        const bool live = r < rows;
                        const float* xrow = p.X + (b0 + (live ? r : 0)) * (long long)X_DIM + IN1_OFF[a];
                        const float* yrow = p.Y + (b0 + (live ? r : 0)) * (long long)Y_DIM + IN2_OFF[b];
#pragma unroll
                        for (int i = 0; i < D1; ++i) xs[q][i] = (live && u < MU) ? __ldg(xrow + u * D1 + i) : 0.f;
#pragma unroll
                        for (int j = 0; j < D2; ++j) ys[q][j] = live ? __ldg(yrow + j) : 0.f;
                    }
                    const bool prof = p.prof && blockIdx.x == 0 && warp == 0 && lane == 0;
                    const long long t0 = prof ? clock64() : 0;
                    if (use > 0) ok = mbar_wait(bars.a_empty + s, (unsigned)((use - 1) & 1), p.status, ERR_TC_A_EMPTY);
                    const long long t1 = prof ? clock64() : 0;
                    if (ok) {
                        unsigned char* hi = smem + TC_OFF_A + s * TC_STAGE_BYTES;
                        unsigned char* lo = hi + TC_STAGE_HALF;
#pragma unroll
                        for (int q = 0; q < RW; ++q) {
                            const int r = warp + q * TC_PRODUCER_WARPS;
                            if (r < rows) {
                                float t[D3];
#pragma unroll
                                for (int k = 0; k < D3; ++k) t[k] = 0.f;
                                float xy = 0.f;
                                sfor<CG_BEGIN[P], CG_BEGIN[P + 1]>([&](auto n_) {
                                    constexpr int N = n_;
                                    if constexpr (N == CG_BEGIN[P] || CG_I[N] != CG_I[N - 1] || CG_J[N] != CG_J[N - 1])
                                        xy = xs[q][CG_I[N]] * ys[q][CG_J[N]];
                                    t[CG_K[N]] = fmaf(xy, (float)CG_V[N], t[CG_K[N]]);
                                });
#pragma unroll
                                for (int k = 0; k < D3; ++k) {
                                    const int off = tc_swizzle(r * D3 + k, lane);
                                    const float th = tf32_hi(t[k]);
                                    *reinterpret_cast<float*>(hi + off) = th;
                                    *reinterpret_cast<float*>(lo + off) = t[k] - th;   // exact; read as TF32 by the MMA
                                }
                            }
                        }
                        fence_async_smem();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(bars.a_full + s);
                        if (prof) {
                            const long long t2 = clock64();
                            atomicAdd(p.prof + 0, (unsigned long long)(t1 - t0));   // wait for the stage
                            atomicAdd(p.prof + 1, (unsigned long long)(t2 - t1));   // loads landing, T, stores
                            atomicAdd(p.prof + 2, 1ull);
                        }
                    }
                    ++stage_it;
                }
            }
        });
    }
    return ok;
}

// ---------------------------------------------------------------------------- MMA issuer (one thread)
template <int O>
__device__ __forceinline__ bool tc_mma_output(const UvwTcParams& p, unsigned char* smem, const TcBars& bars,
                                              long long row_lo, long long row_hi, long long& stage_it, long long& acc_it,
                                              int& w_use, unsigned tmem_base) {
    constexpr int D3 = OUT_D[O];
    constexpr int RPC = 128 / D3;
    constexpr int MW = OUT_MUL[O];
    // Issuing a tcgen05.mma costs about 90 cycles whatever its size, so hi.hi and hi.lo go out as one MMA: the
    // lo tile of the weights follows the hi tile in shared memory, and a B descriptor over 2 MW rows covers
    // both.  The accumulator tile is then [hi.hi + lo.hi | hi.lo], summed by the epilogue.
    constexpr bool WIDE = tc_wide(O);
    constexpr int ACC_COLS = TC_ACC_COLS;
    constexpr int NACC = TC_NACC;
    constexpr unsigned IDESC = tc_instr_desc(MW), IDESC_WIDE = tc_instr_desc(2 * MW);
    constexpr int BLOCK = tc_block_bytes(O);
    if (row_lo >= row_hi) return true;
    // the weights of the previous output must not be overwritten while tensor cores still read them
    if (w_use > 0) {
        tc_commit(bars.w_free);
        if (!mbar_wait(bars.w_free, (unsigned)((w_use - 1) & 1), p.status, ERR_TC_W)) return false;
    }
    mbar_arrive_expect_tx(bars.w_full, (unsigned)tc_w_bytes(O));
    {
        const unsigned char* src = reinterpret_cast<const unsigned char*>(p.Wpacked) + tc_w_offset(O);
        constexpr int TOTAL = tc_w_bytes(O);
        for (int off = 0; off < TOTAL; off += 32768) {
            const int n = TOTAL - off < 32768 ? TOTAL - off : 32768;
            bulk_g2s(smem + TC_OFF_W + off, src + off, (unsigned)n, bars.w_full);
        }
    }
    if (!mbar_wait(bars.w_full, (unsigned)(w_use & 1), p.status, ERR_TC_W)) return false;
    ++w_use;
    const unsigned long long w_desc0 = tc_smem_desc(smem_u32(smem + TC_OFF_W));
    const unsigned long long a_desc0 = tc_smem_desc(smem_u32(smem + TC_OFF_A));
    bool ok = true;
    for (long long b0 = row_lo; b0 < row_hi && ok; b0 += RPC) {
        const int t = (int)(acc_it % NACC);
        const long long acc_use = acc_it / NACC;
        if (acc_use > 0) ok = mbar_wait(bars.acc_empty + t, (unsigned)((acc_use - 1) & 1), p.status, ERR_TC_ACC_EMPTY);
        if (!ok) break;
        tc_fence_after();
        const unsigned tmem_d = tmem_base + (unsigned)(t * ACC_COLS);
        unsigned accumulate = 0;
        sfor<0, N_INSTR>([&](auto p_) {
            constexpr int P = p_;
            if constexpr (I_OUT[P] == O) {
                for (int h = 0; h < tc_khalves(P) && ok; ++h) {
                    const int s = (int)(stage_it % TC_NA);
                    const long long use = stage_it / TC_NA;
                    const bool prof = p.prof && blockIdx.x == 0;
                    const long long t0 = prof ? clock64() : 0;
                    ok = mbar_wait(bars.a_full + s, (unsigned)(use & 1), p.status, ERR_TC_A_FULL);
                    const long long t1 = prof ? clock64() : 0;
                    if (ok) {
                        tc_fence_after();
                        // descriptors differ from the base ones only in the start-address field (16-byte units):
                        // one add per operand instead of rebuilding them (the issuing thread is latency bound)
                        const unsigned long long da_hi = a_desc0 + (unsigned long long)((s * TC_STAGE_BYTES) >> 4);
                        const unsigned long long da_lo = da_hi + (TC_STAGE_HALF >> 4);
                        const unsigned long long db_hi = w_desc0 + (unsigned long long)(((tc_blocks_before(O, P) + h) * 2 * BLOCK) >> 4);
                        const unsigned long long db_lo = db_hi + (BLOCK >> 4);
#pragma unroll
                        for (int kk = 0; kk < 4; ++kk) {
                            if constexpr (WIDE) {
                                tc_mma(tmem_d, da_hi + 2 * kk, db_hi + 2 * kk, IDESC_WIDE, accumulate);
                            } else {
                                tc_mma(tmem_d, da_hi + 2 * kk, db_hi + 2 * kk, IDESC, accumulate);
                                tc_mma(tmem_d, da_hi + 2 * kk, db_lo + 2 * kk, IDESC, 1);
                            }
                            accumulate = 1;
                            tc_mma(tmem_d, da_lo + 2 * kk, db_hi + 2 * kk, IDESC, 1);
                        }
                        tc_commit(bars.a_empty + s);   // the stage may be refilled once these MMAs have read it
                        if (prof) {
                            atomicAdd(p.prof + 8, (unsigned long long)(t1 - t0));             // wait for operands
                            atomicAdd(p.prof + 9, (unsigned long long)(clock64() - t1));      // issue
                        }
                    }
                    ++stage_it;
                }
            }
        });
        if (ok) tc_commit(bars.acc_full + t);
        ++acc_it;
    }
    return ok;
}

// ---------------------------------------------------------------------------- epilogue warps
// AND-reduction of a flag over the epilogue warps (hardware barrier 1).
__device__ __forceinline__ bool tc_epilogue_all(bool ok) {
    unsigned r;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\tsetp.ne.b32 q, %1, 0;\n\t"
        "bar.red.and.pred p, 1, %2, q;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(r)
        : "r"((unsigned)ok), "n"(TC_EPILOGUE_WARPS * 32)
        : "memory");
    return r != 0;
}

template <int O>
__device__ __forceinline__ bool tc_epilogue_output(const UvwTcParams& p, unsigned char* smem, const TcBars& bars,
                                                   long long row_lo, long long row_hi, long long& acc_it,
                                                   unsigned tmem_base, int ewarp, int lane) {
    constexpr int D3 = OUT_D[O];
    constexpr int RPC = 128 / D3;
    constexpr int MW = OUT_MUL[O];
    constexpr bool WIDE = tc_wide(O);
    constexpr int ACC_COLS = TC_ACC_COLS;
    constexpr int NACC = TC_NACC;
    float* stg = reinterpret_cast<float*>(smem + TC_OFF_STG);
    const int et = ewarp * 32 + lane;
    bool ok = true;
    for (long long b0 = row_lo; b0 < row_hi && ok; b0 += RPC) {
        const int rows = (int)(row_hi - b0 < RPC ? row_hi - b0 : RPC);
        const int t = (int)(acc_it % NACC);
        const long long use = acc_it / NACC;
        const bool prof = p.prof && blockIdx.x == 0 && et == 0;
        const long long t0 = prof ? clock64() : 0;
        ok = mbar_wait(bars.acc_full + t, (unsigned)(use & 1), p.status, ERR_TC_ACC_FULL);
        if (prof) atomicAdd(p.prof + 16, (unsigned long long)(clock64() - t0));
        const long long t1 = prof ? clock64() : 0;
        // the four warps must agree before anyone touches the staging buffer or skips a barrier
        ok = tc_epilogue_all(ok);
        if (!ok) break;
        tc_fence_after();
        // (ewarp is the warp's TMEM lane quarter) accumulator row m = 32 * ewarp + lane holds (row m / D3, component m % D3) for all w
        const unsigned taddr = tmem_base + ((unsigned)(ewarp * 32) << 16) + (unsigned)(t * ACC_COLS);
#pragma unroll
        for (int c0 = 0; c0 < MW; c0 += 16) {
            unsigned v[16], v2[16];
            tc_load16(taddr + (unsigned)c0, v);
            if constexpr (WIDE) tc_load16(taddr + (unsigned)(MW + c0), v2);   // the hi.lo half of the tile
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
            for (int c = 0; c < 16; ++c) {
                float val = __uint_as_float(v[c]);
                if constexpr (WIDE) val += __uint_as_float(v2[c]);
                stg[(ewarp * 32 + lane) * TC_STG_PITCH + c0 + c] = val;
            }
        }
        tc_fence_before();
        asm volatile("bar.sync 1, %0;" ::"n"(TC_EPILOGUE_WARPS * 32) : "memory");
        if (et == 0) mbar_arrive(bars.acc_empty + t);   // the accumulator tile may be overwritten
        // staged rows (row * D3 + k) x w  ->  Z[row][OUT_OFF + w * D3 + k], contiguous per batch row
        constexpr int ROWLEN = MW * D3;
        for (int e = et; e < rows * ROWLEN; e += TC_EPILOGUE_WARPS * 32) {
            const int r = e / ROWLEN, j = e - r * ROWLEN;
            const int w = j / D3, k = j - w * D3;
            p.Z[(b0 + r) * (long long)Z_DIM + OUT_OFF[O] + j] = stg[(r * D3 + k) * TC_STG_PITCH + w];
        }
        asm volatile("bar.sync 1, %0;" ::"n"(TC_EPILOGUE_WARPS * 32) : "memory");
        if (prof) {
            atomicAdd(p.prof + 17, (unsigned long long)(clock64() - t1));
            atomicAdd(p.prof + 18, 1ull);
        }
        ++acc_it;
    }
    return ok;
}

constexpr bool tc_output_has_paths(int o) {
    for (int p = 0; p < N_INSTR; ++p)
        if (I_OUT[p] == o) return true;
    return false;
}

__device__ void uvw_tc_forward(const UvwTcParams& p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    // the 128-byte swizzle pattern repeats every 1024 bytes: operand tiles must start on that boundary
    unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    const TcBars bars(smem);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    long long row_lo, row_hi;
    tc_row_range(p.batch, row_lo, row_hi);

    if (tid == 0) {
        for (int i = 0; i < TC_NA; ++i) {
            mbar_init(bars.a_full + i, TC_PRODUCER_WARPS);
            mbar_init(bars.a_empty + i, 1);
        }
        for (int i = 0; i < TC_MAX_ACC; ++i) {
            mbar_init(bars.acc_full + i, 1);
            mbar_init(bars.acc_empty + i, 1);
        }
        mbar_init(bars.w_full, 1);
        mbar_init(bars.w_free, 1);
        fence_mbar_init();
    }
    if (warp == TC_PRODUCER_WARPS) {   // the MMA warp owns the tensor memory allocation
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(bars.tmem_slot)),
                     "n"(TC_TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem_base = *reinterpret_cast<volatile unsigned*>(bars.tmem_slot);

    if (warp < TC_PRODUCER_WARPS) {
        long long stage_it = 0;
        bool ok = true;
        sfor<0, N_OUT>([&](auto o_) {
            constexpr int O = o_;
            if constexpr (tc_output_has_paths(O)) {
                if (ok) ok = tc_produce_output<O>(p, smem, bars, row_lo, row_hi, stage_it, warp, lane);
            } else {
                // an output irrep that no path writes is zero
                for (long long b = row_lo + warp; b < row_hi; b += TC_PRODUCER_WARPS)
                    for (int j = lane; j < OUT_MUL[O] * OUT_D[O]; j += 32) p.Z[b * (long long)Z_DIM + OUT_OFF[O] + j] = 0.f;
            }
        });
    } else if (warp == TC_PRODUCER_WARPS) {
        if (lane == 0) {
            long long stage_it = 0, acc_it = 0;
            int w_use = 0;
            bool ok = true;
            sfor<0, N_OUT>([&](auto o_) {
                constexpr int O = o_;
                if constexpr (tc_output_has_paths(O)) {
                    if (ok) ok = tc_mma_output<O>(p, smem, bars, row_lo, row_hi, stage_it, acc_it, w_use, tmem_base);
                }
            });
        }
        __syncwarp();
    } else {
        long long acc_it = 0;
        bool ok = true;
        sfor<0, N_OUT>([&](auto o_) {
            constexpr int O = o_;
            if constexpr (tc_output_has_paths(O)) {
                // a warp may only read the TMEM lanes of its own quarter: 32 * (warp index mod 4)
                if (ok) ok = tc_epilogue_output<O>(p, smem, bars, row_lo, row_hi, acc_it, tmem_base, warp & 3, lane);
            }
        });
    }
    tc_fence_before();
    __syncthreads();
    if (warp == TC_PRODUCER_WARPS) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "n"(TC_TMEM_COLS) : "memory");
    }
}

}  // namespace oeq

#define OEQ_K_UVW_TC_FWD 20

extern "C" __global__ void __launch_bounds__(oeq::TC_THREADS, 1) oeq_uvw_tc_kernel(const oeq::UvwTcParams p) {
    oeq::uvw_tc_forward(p);
}

// Splits the shared weights into TF32 hi / lo parts and lays them out as the B operand of the MMA:
// per output irrep, per path into it, per 32-wide slice of u, a [mul_out x 32] K-major tile with the
// 128-byte swizzle for hi and one for lo.  Rows of u beyond the multiplicity are zero.
extern "C" __global__ void oeq_uvw_pack_weights(const float* __restrict__ W, float* __restrict__ packed) {
    using namespace oeqd;
    const int tid = blockIdx.x * blockDim.x + threadIdx.x, nthreads = gridDim.x * blockDim.x;
    oeq::sfor<0, N_INSTR>([&](auto p_) {
        constexpr int P = p_;
        constexpr int O = I_OUT[P], MU = IN1_MUL[I_IN1[P]], MW = OUT_MUL[O];
        constexpr int KH = oeq::tc_khalves(P), BLOCK = oeq::tc_block_bytes(O);
        unsigned char* base = reinterpret_cast<unsigned char*>(packed) + oeq::tc_w_offset(O) +
                              oeq::tc_blocks_before(O, P) * 2 * BLOCK;
        for (int e = tid; e < KH * MW * 32; e += nthreads) {
            const int col = e & 31, w = (e >> 5) % MW, h = e / (32 * MW);
            const int u = h * 32 + col;
            float v = 0.f;
            if (u < MU) {
                // kernel weight order: 32-wide (u, w) chunks, u-chunk major, each chunk [u][w] (v == 1)
                const int uc = u >> 5, ul = u & 31, wc = w >> 5, wl = w & 31;
                const int ulen = (MU - (uc << 5)) < 32 ? (MU - (uc << 5)) : 32;
                const int wlen = (MW - (wc << 5)) < 32 ? (MW - (wc << 5)) : 32;
                v = W[W_OFF[P] + (uc << 5) * MW + ulen * (wc << 5) + ul * wlen + wl];
            }
            const float hi = oeq::tf32_round(v), lo = oeq::tf32_round(v - hi);
            unsigned char* blk = base + h * 2 * BLOCK;
            *reinterpret_cast<float*>(blk + oeq::tc_swizzle(w, col)) = hi;
            *reinterpret_cast<float*>(blk + BLOCK + oeq::tc_swizzle(w, col)) = lo;
        }
    });
}
