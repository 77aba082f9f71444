// "uvu" tensor product kernels for sm_100a: batch rows, and the fused
// gather - tensor product - scatter graph convolution (deterministic segmented
// reduction over sorted edges, or atomic accumulation for arbitrary order).
//
// Replaces the reference's generated kernels
// (openequivariance/templates/loop_unroll_batch.cuh:24-133,
//  loop_unroll_tp.cuh:20-252, loop_unroll_conv_atomic.cuh:40-141,
//  loop_unroll_conv_det.cuh:33-222) with one hand-written template that is
// specialised by a constexpr problem descriptor (namespace oeqd).
//
// Execution model
//   * An "item" is one batch row or one graph edge.  A "group" of
//     G = MULG * PS threads works on one item at a time: thread (part, u)
//     owns channel u of the instructions assigned to partition `part`.
//   * A CTA holds NG groups plus one producer warp.  The producer warp stages
//     every item's rows (X gathered by sender index, Y, per-item W, and dZ
//     gathered by receiver index in the backward pass) into a ring of shared
//     memory stages with 1-D bulk async copies (TMA) that complete on an
//     mbarrier; rows that break the 16-byte rule fall back to cp.async.
//   * Clebsch-Gordan coefficients times path weights are compile-time
//     constants; the contraction is fully unrolled straight-line FMA code.
//   * Deterministic convolution: every group owns a contiguous, node-aligned
//     slice of the sorted edge list, accumulates a node's sum in registers
//     and writes each output row exactly once (rows without edges are written
//     as zeros), so no scratch buffer or fix-up pass exists.
//   * All waits are bounded; a wait that runs out sets *status and the CTA
//     drains its copies and returns.
#pragma once
#include "oeq_common.cuh"

namespace oeq {
using namespace oeqd;

struct UvuParams {
    const T* X;
    const T* Y;
    const T* W;
    T* Z;          // forward output
    const T* dZ;   // backward input
    T* dX;
    T* dY;
    T* dW;
    const long long* rows;  // receiver of each edge
    const long long* cols;  // sender of each edge
    const long long* perm;  // deterministic backward: k-th edge in (sender, receiver) order
    long long n_items;      // batch rows or edges
    long long n_nodes;
    T* ws;                  // scratch: per-group partial sums of shared-weight gradients
    int* status;
    int stages;             // shared-memory stages per group
    int flags;              // bit0 X bulk-able, bit1 Y, bit2 W, bit3 Z/dZ, bit4 dX rows bulk-able
};

constexpr int MODE_BATCH = 0;
constexpr int MODE_DET = 1;
constexpr int MODE_ATOMIC = 2;

constexpr int G = MULG * PS;
constexpr int NCONSUMERS = NG * G;
constexpr int NTHREADS = NCONSUMERS + 32;
constexpr int WARPS_PER_GROUP = G / 32;

// ---------------------------------------------------------------- helpers on the descriptor

__host__ __device__ constexpr int pad16(int bytes) { return (bytes + 15) / 16 * 16; }
constexpr int ELEM = sizeof(T);
constexpr int XB = pad16(X_DIM * ELEM), YB = pad16(Y_DIM * ELEM), ZB = pad16(Z_DIM * ELEM);
constexpr int WB = SHARED_W ? 0 : pad16(W_NUMEL * ELEM);
constexpr int SWB = SHARED_W ? pad16(W_NUMEL * ELEM) : 0;

template <bool BWD>
struct StageLayout {
    static constexpr int OFF_X = 0;
    static constexpr int OFF_Y = OFF_X + XB;
    static constexpr int OFF_W = OFF_Y + YB;
    static constexpr int OFF_DZ = OFF_W + WB;
    static constexpr int BYTES = OFF_DZ + (BWD ? ZB : 0);
};

constexpr bool fwd_part_uses_in1(int q, int a) {
    for (int p = 0; p < N_INSTR; ++p)
        if (FWD_PART_OF_OUT[I_OUT[p]] == q && I_IN1[p] == a) return true;
    return false;
}
constexpr bool bwd_part_uses_in1(int q, int a) {
    for (int p = 0; p < N_INSTR; ++p)
        if (BWD_PART_OF_INSTR[p] == q && I_IN1[p] == a) return true;
    return false;
}
constexpr bool any_part_uses_in1(int a) {
    for (int p = 0; p < N_INSTR; ++p)
        if (I_IN1[p] == a) return true;
    return false;
}
constexpr bool all_in2_mul_one() {
    for (int p = 0; p < N_INSTR; ++p)
        if (IN2_MUL[I_IN2[p]] != 1) return false;
    return true;
}
constexpr int CHANNELS = MULG * NCH;

// Offset of weight (u, v) of instruction P in the kernel weight layout: the
// multiplicity axes are cut into 32-wide chunks, chunks are ordered u-chunk
// major, and each chunk is stored [v][u].
template <int P>
__device__ __forceinline__ int weight_offset(int u, int v) {
    constexpr int M1 = IN1_MUL[I_IN1[P]];
    constexpr int M2 = IN2_MUL[I_IN2[P]];
    if constexpr (M2 == 1 || (M1 <= 32 && M2 <= 32)) {
        return W_OFF[P] + v * M1 + u;
    } else {
        const int uc = u >> 5, ul = u & 31, vc = v >> 5, vl = v & 31;
        const int ulen = (M1 - (uc << 5)) < 32 ? (M1 - (uc << 5)) : 32;
        return W_OFF[P] + (uc << 5) * M2 + ulen * (vc << 5) + vl * ulen + ul;
    }
}

// t[k] += sum_n c_n * x[i_n] * y[j_n] over the nonzeros of instruction P.
template <int P, class XA, class YA, class TA>
__device__ __forceinline__ void cg_forward(const XA& x, const YA& y, TA& t) {
    sfor<CG_BEGIN[P], CG_BEGIN[P + 1]>([&](auto n) {
        constexpr int N = n;
        t[CG_K[N]] = fma(x[CG_I[N]] * y[CG_J[N]], (T)CG_V[N], t[CG_K[N]]);
    });
}

// Backward of the above for one (u, v): with g = dZ block of the channel,
//   dxl[i] += c g[k] y[j];  dyl[j] += c g[k] x[i];  returns sum c g[k] x[i] y[j].
template <int P, class XA, class YA, class GA, class DXA, class DYA>
__device__ __forceinline__ T cg_backward(const XA& x, const YA& y, const GA& g, DXA& dxl, DYA& dyl) {
    T tw = (T)0;
    sfor<CG_BEGIN[P], CG_BEGIN[P + 1]>([&](auto n) {
        constexpr int N = n;
        const T q = (T)CG_V[N] * g[CG_K[N]];
        const T qx = q * x[CG_I[N]];
        dxl[CG_I[N]] = fma(q, y[CG_J[N]], dxl[CG_I[N]]);
        dyl[CG_J[N]] += qx;
        tw = fma(qx, y[CG_J[N]], tw);
    });
    return tw;
}

// ---------------------------------------------------------------- shared memory map

template <bool BWD, int MODE>
struct Smem {
    using L = StageLayout<BWD>;
    // per-group extras
    static constexpr int ZBUF = (!BWD && MODE == MODE_BATCH) ? 2 * ZB : 0;      // staged output rows
    static constexpr int DXBUF = BWD ? PS * XB : 0;                             // dX partials per partition
    static constexpr int DYSLOT = BWD ? 2 * WARPS_PER_GROUP * YB : 0;           // per-warp dY partials, double buffered
    static constexpr int DWACC = (BWD && SHARED_W) ? pad16(W_NUMEL * ELEM) : 0; // shared-weight gradient
    static constexpr int EXTRA = ZBUF + DXBUF + DYSLOT + DWACC;

    unsigned char* base;
    int stages;
    __device__ Smem(unsigned char* b, int s) : base(b), stages(s) {}
    __device__ unsigned long long* full(int g, int s) const {
        return reinterpret_cast<unsigned long long*>(base) + (g * stages + s) * 2;
    }
    __device__ unsigned long long* empty(int g, int s) const { return full(g, s) + 1; }
    __device__ long long* hdr(int g, int s) const {
        return reinterpret_cast<long long*>(base + NG * stages * 16) + (g * stages + s) * 4;
    }
    __device__ long long* bounds() const {  // [0..NG] edge bounds, [NG+1 .. 2NG+1] node bounds
        return reinterpret_cast<long long*>(base + NG * stages * 48);
    }
    __device__ unsigned char* shared_w() const { return base + NG * stages * 48 + pad16((2 * NG + 2) * 8); }
    __device__ unsigned char* group_base(int g) const {
        return shared_w() + SWB + (long long)g * (stages * L::BYTES + EXTRA);
    }
    __device__ unsigned char* stage(int g, int s) const { return group_base(g) + s * L::BYTES; }
    __device__ unsigned char* extra(int g) const { return group_base(g) + stages * L::BYTES; }
};

// ---------------------------------------------------------------- producer warp

template <int MODE, bool BWD>
__device__ __forceinline__ long long item_key(const UvuParams& p, long long k) {
    // value whose runs define a segment: receiver (forward) or sender (backward)
    if constexpr (!BWD) {
        return p.rows[k];
    } else {
        return MODE == MODE_DET ? p.cols[p.perm[k]] : p.cols[k];
    }
}

// First index >= t that starts a new run of item_key (warp-cooperative).
template <int MODE, bool BWD>
__device__ long long align_forward(const UvuParams& p, long long t, int lane) {
    const long long n = p.n_items;
    if (t <= 0) return 0;
    if (t >= n) return n;
    for (long long base = t; base < n + 32; base += 32) {
        const long long idx = base + lane;
        bool boundary = idx >= n;
        if (!boundary) boundary = item_key<MODE, BWD>(p, idx) != item_key<MODE, BWD>(p, idx - 1);
        const unsigned ballot = __ballot_sync(0xffffffffu, boundary);
        if (ballot) return base + (__ffs(ballot) - 1);
    }
    return n;
}

template <int MODE, bool BWD>
__device__ void producer(const UvuParams& p, const Smem<BWD, MODE>& sm, int lane) {
    using L = StageLayout<BWD>;
    const int S = sm.stages;
    const long long total_groups = (long long)gridDim.x * NG;
    const long long gid0 = (long long)blockIdx.x * NG;
    const bool xb = p.flags & 1, yb = p.flags & 2, wb = p.flags & 4, zb = p.flags & 8;
    const long long* bnd = sm.bounds();

    long long first[NG], count[NG];
#pragma unroll
    for (int g = 0; g < NG; ++g) {
        if constexpr (MODE == MODE_BATCH) {
            first[g] = gid0 + g;
            count[g] = first[g] < p.n_items ? (p.n_items - first[g] + total_groups - 1) / total_groups : 0;
        } else {
            first[g] = bnd[g];
            count[g] = bnd[g + 1] - bnd[g];
        }
    }
    long long max_count = 0;
#pragma unroll
    for (int g = 0; g < NG; ++g) max_count = count[g] > max_count ? count[g] : max_count;

    // per-lane prefetched indices of a block of 32 items, per group
    long long ie[NG], is_[NG], ir[NG];
    bool ok = true;
    for (long long it = 0; it < max_count && ok; ++it) {
#pragma unroll
        for (int g = 0; g < NG; ++g) {
            if (it >= count[g] || !ok) continue;
            const int stage = (int)(it % S);
            const long long use = it / S;
            if constexpr (MODE != MODE_BATCH) {
                if ((it & 31) == 0) {
                    const long long k = first[g] + it + lane;
                    long long e = 0, s = 0, r = 0;
                    if (k < first[g] + count[g]) {
                        e = (BWD && MODE == MODE_DET) ? p.perm[k] : k;
                        s = p.cols[e];
                        r = p.rows[e];
                    }
                    ie[g] = e; is_[g] = s; ir[g] = r;
                }
            }
            long long e, s, r;
            if constexpr (MODE == MODE_BATCH) {
                e = s = r = first[g] + it * total_groups;
            } else {
                const int src = (int)(it & 31);
                e = __shfl_sync(0xffffffffu, ie[g], src);
                s = __shfl_sync(0xffffffffu, is_[g], src);
                r = __shfl_sync(0xffffffffu, ir[g], src);
            }
            if (use > 0) {
                if (!mbar_wait(sm.empty(g, stage), (unsigned)((use - 1) & 1), p.status, ERR_WAIT_EMPTY)) {
                    ok = false;
                    continue;
                }
            }
            unsigned char* st = sm.stage(g, stage);
            unsigned long long* full = sm.full(g, stage);
            const T* xsrc = p.X + s * X_DIM;
            const T* ysrc = p.Y + e * Y_DIM;
            const T* wsrc = SHARED_W ? nullptr : p.W + e * (long long)W_NUMEL;
            const T* zsrc = BWD ? p.dZ + r * (long long)Z_DIM : nullptr;
            if (lane == 0) {
                long long* h = sm.hdr(g, stage);
                h[0] = e; h[1] = s; h[2] = r;
                unsigned bytes = 0;
                if (xb) bytes += XB;
                if (yb) bytes += YB;
                if (wb && !SHARED_W) bytes += WB;
                if (BWD && zb) bytes += ZB;
                mbar_arrive_expect_tx(full, bytes);
                if (xb) bulk_g2s(st + L::OFF_X, xsrc, XB, full);
                if (yb) bulk_g2s(st + L::OFF_Y, ysrc, YB, full);
                if (wb && !SHARED_W) bulk_g2s(st + L::OFF_W, wsrc, WB, full);
                if (BWD && zb) bulk_g2s(st + L::OFF_DZ, zsrc, ZB, full);
            }
            const bool any_elem = !xb || !yb || (!wb && !SHARED_W) || (BWD && !zb);
            if (any_elem) {
                if (!xb) for (int i = lane; i < X_DIM; i += 32) cp_async_elem<ELEM>((T*)(st + L::OFF_X) + i, xsrc + i);
                if (!yb) for (int i = lane; i < Y_DIM; i += 32) cp_async_elem<ELEM>((T*)(st + L::OFF_Y) + i, ysrc + i);
                if constexpr (!SHARED_W) {
                    if (!wb) for (int i = lane; i < W_NUMEL; i += 32) cp_async_elem<ELEM>((T*)(st + L::OFF_W) + i, wsrc + i);
                }
                if constexpr (BWD) {
                    if (!zb) for (int i = lane; i < Z_DIM; i += 32) cp_async_elem<ELEM>((T*)(st + L::OFF_DZ) + i, zsrc + i);
                }
                cp_async_arrive_noinc(full);
            }
        }
    }
    if (!ok) {
        // a consumer stopped releasing stages: let the copies already issued land, then leave
        asm volatile("cp.async.wait_all;" ::: "memory");
    }
}

// ---------------------------------------------------------------- consumer: forward

template <int Q, int C, class ZA>
__device__ __forceinline__ void forward_item(const T* __restrict__ sX, const T* __restrict__ sY,
                                             const T* __restrict__ sWt, int u, ZA& zacc) {
    // registers: the channel's inputs for every first-input irrep this partition reads
    T xr[XPC];
    sfor<0, N_IN1>([&](auto a_) {
        constexpr int a = a_;
        if constexpr (fwd_part_uses_in1(Q, a)) {
            const bool live = (IN1_MUL[a] == CHANNELS) || (u < IN1_MUL[a]);
#pragma unroll
            for (int i = 0; i < IN1_D[a]; ++i) xr[XR_OFF[a] + i] = live ? sX[IN1_OFF[a] + u * IN1_D[a] + i] : (T)0;
        }
    });
    sfor<0, N_OUT>([&](auto o_) {
        constexpr int o = o_;
        if constexpr (FWD_PART_OF_OUT[o] == Q) {
            constexpr int D3 = OUT_D[o];
            T acc[D3];
#pragma unroll
            for (int k = 0; k < D3; ++k) acc[k] = (T)0;
            sfor<0, N_INSTR>([&](auto p_) {
                constexpr int P = p_;
                if constexpr (I_OUT[P] == o) {
                    constexpr int a = I_IN1[P], b = I_IN2[P];
                    constexpr int D1 = IN1_D[a], D2 = IN2_D[b], M2 = IN2_MUL[b];
                    if ((IN1_MUL[a] == CHANNELS) || (u < IN1_MUL[a])) {
                        const T* x = xr + XR_OFF[a];
                        if constexpr (M2 == 1) {
                            T y[D2];
#pragma unroll
                            for (int j = 0; j < D2; ++j) y[j] = sY[IN2_OFF[b] + j];
                            T t[D3];
#pragma unroll
                            for (int k = 0; k < D3; ++k) t[k] = (T)0;
                            cg_forward<P>(x, y, t);
                            const T w = sWt[weight_offset<P>(u, 0)];
#pragma unroll
                            for (int k = 0; k < D3; ++k) acc[k] = fma(w, t[k], acc[k]);
                        } else {
#pragma unroll 1
                            for (int v = 0; v < M2; ++v) {
                                T y[D2];
#pragma unroll
                                for (int j = 0; j < D2; ++j) y[j] = sY[IN2_OFF[b] + v * D2 + j];
                                T t[D3];
#pragma unroll
                                for (int k = 0; k < D3; ++k) t[k] = (T)0;
                                cg_forward<P>(x, y, t);
                                const T w = sWt[weight_offset<P>(u, v)];
#pragma unroll
                                for (int k = 0; k < D3; ++k) acc[k] = fma(w, t[k], acc[k]);
                            }
                        }
                    }
                }
            });
#pragma unroll
            for (int k = 0; k < D3; ++k) zacc[C * ZPC_MAX + ZR_OFF[o] + k] += acc[k];
        }
    });
}

// Visit every (output irrep, k) register of partition Q / channel chunk C.
template <int Q, int C, class F>
__device__ __forceinline__ void for_each_out(int u, F&& f) {
    sfor<0, N_OUT>([&](auto o_) {
        constexpr int o = o_;
        if constexpr (FWD_PART_OF_OUT[o] == Q) {
            if ((OUT_MUL[o] == CHANNELS) || (u < OUT_MUL[o])) {
#pragma unroll
                for (int k = 0; k < OUT_D[o]; ++k) f(OUT_OFF[o] + u * OUT_D[o] + k, C * ZPC_MAX + ZR_OFF[o] + k);
            }
        }
    });
}

template <int MODE>
__device__ void consumer_forward(const UvuParams& p, const Smem<false, MODE>& sm, int g, int tg) {
    using L = StageLayout<false>;
    const int S = sm.stages;
    const int part = tg / MULG;
    const int u0 = tg % MULG;
    const long long total_groups = (long long)gridDim.x * NG;
    const long long gid = (long long)blockIdx.x * NG + g;
    const long long* bnd = sm.bounds();
    const int bar_id = 1 + g;

    long long count;
    if constexpr (MODE == MODE_BATCH) {
        count = gid < p.n_items ? (p.n_items - gid + total_groups - 1) / total_groups : 0;
    } else {
        count = bnd[g + 1] - bnd[g];
    }
    const T* sWshared = reinterpret_cast<const T*>(sm.shared_w());
    T* zbuf = reinterpret_cast<T*>(sm.extra(g));
    const bool z_bulk = p.flags & 8;

    T zacc[ZPC_MAX * NCH];
#pragma unroll
    for (int i = 0; i < ZPC_MAX * NCH; ++i) zacc[i] = (T)0;

    // Finish the output row of node `node`: store (or atomically add) and clear the registers.
    auto flush = [&](long long node) {
        T* zrow = p.Z + node * (long long)Z_DIM;
        sfor<0, PS>([&](auto q_) {
            constexpr int Q = q_;
            if (part == Q) {
                sfor<0, NCH>([&](auto c_) {
                    constexpr int C = c_;
                    for_each_out<Q, C>(u0 + C * MULG, [&](int zoff, int reg) {
                        if constexpr (MODE == MODE_DET) zrow[zoff] = zacc[reg];
                        else red_add(zrow + zoff, zacc[reg]);
                        zacc[reg] = (T)0;
                    });
                });
            }
        });
    };
    auto zero_nodes = [&](long long lo, long long hi) {
        for (long long node = lo; node < hi; ++node) {
            T* zrow = p.Z + node * (long long)Z_DIM;
            for (int i = tg; i < Z_DIM; i += G) zrow[i] = (T)0;
        }
    };

    long long prev = -1;
    long long next_unwritten = 0;  // deterministic mode: first node of this group's range not yet written
    if constexpr (MODE == MODE_DET) next_unwritten = bnd[NG + 1 + g];
    bool ok = true;

    for (long long it = 0; it < count; ++it) {
        const int stage = (int)(it % S);
        const long long use = it / S;
        if (!mbar_wait(sm.full(g, stage), (unsigned)(use & 1), p.status, ERR_WAIT_FULL)) {
            ok = false;
            break;
        }
        const unsigned char* st = sm.stage(g, stage);
        const long long* h = sm.hdr(g, stage);
        const long long node = h[2];
        if constexpr (MODE != MODE_BATCH) {
            if (prev >= 0 && node != prev) {
                flush(prev);
                if constexpr (MODE == MODE_DET) next_unwritten = prev + 1;
            }
            if constexpr (MODE == MODE_DET) {
                if (node != prev && next_unwritten < node) zero_nodes(next_unwritten, node);
            }
            prev = node;
        }
        const T* sX = reinterpret_cast<const T*>(st + L::OFF_X);
        const T* sY = reinterpret_cast<const T*>(st + L::OFF_Y);
        const T* sWt = SHARED_W ? sWshared : reinterpret_cast<const T*>(st + L::OFF_W);
        sfor<0, PS>([&](auto q_) {
            constexpr int Q = q_;
            if (part == Q) {
                sfor<0, NCH>([&](auto c_) {
                    constexpr int C = c_;
                    forward_item<Q, C>(sX, sY, sWt, u0 + C * MULG, zacc);
                });
            }
        });
        mbar_arrive(sm.empty(g, stage));

        if constexpr (MODE == MODE_BATCH) {
            T* zb = zbuf + (it & 1) * (ZB / ELEM);
            // the bulk store that last read this buffer (two items ago) must be done
            if (tg == 0) bulk_wait_read<1>();
            group_sync(bar_id, G);
            sfor<0, PS>([&](auto q_) {
                constexpr int Q = q_;
                if (part == Q) {
                    sfor<0, NCH>([&](auto c_) {
                        constexpr int C = c_;
                        for_each_out<Q, C>(u0 + C * MULG, [&](int zoff, int reg) {
                            zb[zoff] = zacc[reg];
                            zacc[reg] = (T)0;
                        });
                    });
                }
            });
            T* zrow = p.Z + node * (long long)Z_DIM;
            if (z_bulk) {
                fence_async_smem();
                group_sync(bar_id, G);
                if (tg == 0) {
                    bulk_s2g(zrow, zb, ZB);
                    bulk_commit();
                }
            } else {
                group_sync(bar_id, G);
                for (int i = tg; i < Z_DIM; i += G) zrow[i] = zb[i];
            }
        }
    }
    if constexpr (MODE != MODE_BATCH) {
        if (ok && prev >= 0) {
            flush(prev);
            if constexpr (MODE == MODE_DET) next_unwritten = prev + 1;
        }
        if constexpr (MODE == MODE_DET) {
            if (ok) zero_nodes(next_unwritten, bnd[NG + 2 + g]);
        }
    }
    if constexpr (MODE == MODE_BATCH) {
        if (tg == 0) bulk_wait_all<0>();
    }
}

// ---------------------------------------------------------------- consumer: backward

template <int Q, int C, class DXA, class DYA>
__device__ __forceinline__ void backward_item(const T* __restrict__ sX, const T* __restrict__ sY,
                                              const T* __restrict__ sWt, const T* __restrict__ sdZ, int u,
                                              long long item, const UvuParams& p, T* __restrict__ dw_acc,
                                              T* __restrict__ dy_slot, int lane, DXA& dxacc, DYA& dyreg) {
    T xr[XPC];
    sfor<0, N_IN1>([&](auto a_) {
        constexpr int a = a_;
        if constexpr (bwd_part_uses_in1(Q, a)) {
            const bool live = (IN1_MUL[a] == CHANNELS) || (u < IN1_MUL[a]);
#pragma unroll
            for (int i = 0; i < IN1_D[a]; ++i) xr[XR_OFF[a] + i] = live ? sX[IN1_OFF[a] + u * IN1_D[a] + i] : (T)0;
        }
    });
    sfor<0, N_INSTR>([&](auto p_) {
        constexpr int P = p_;
        if constexpr (BWD_PART_OF_INSTR[P] == Q) {
            constexpr int a = I_IN1[P], b = I_IN2[P], o = I_OUT[P];
            constexpr int D1 = IN1_D[a], D2 = IN2_D[b], D3 = OUT_D[o], M2 = IN2_MUL[b];
            const bool live = (IN1_MUL[a] == CHANNELS) || (u < IN1_MUL[a]);
            T gz[D3];
#pragma unroll
            for (int k = 0; k < D3; ++k) gz[k] = live ? sdZ[OUT_OFF[o] + u * D3 + k] : (T)0;
            const T* x = xr + XR_OFF[a];
            T dxl[D1];
#pragma unroll
            for (int i = 0; i < D1; ++i) dxl[i] = (T)0;
            if constexpr (M2 == 1) {
                T y[D2], dyl[D2];
#pragma unroll
                for (int j = 0; j < D2; ++j) { y[j] = sY[IN2_OFF[b] + j]; dyl[j] = (T)0; }
                const T w = live ? sWt[weight_offset<P>(u, 0)] : (T)0;
                const T tw = cg_backward<P>(x, y, gz, dxl, dyl);
                if (live) {
                    if constexpr (SHARED_W) dw_acc[weight_offset<P>(u, 0)] += tw;
                    else p.dW[item * (long long)W_NUMEL + weight_offset<P>(u, 0)] = tw;
                }
#pragma unroll
                for (int i = 0; i < D1; ++i) dxacc[C * XPC + XR_OFF[a] + i] = fma(w, dxl[i], dxacc[C * XPC + XR_OFF[a] + i]);
#pragma unroll
                for (int j = 0; j < D2; ++j) dyreg[IN2_OFF[b] + j] = fma(w, dyl[j], dyreg[IN2_OFF[b] + j]);
            } else {
#pragma unroll 1
                for (int v = 0; v < M2; ++v) {
                    T y[D2], dyl[D2], dxv[D1];
#pragma unroll
                    for (int j = 0; j < D2; ++j) { y[j] = sY[IN2_OFF[b] + v * D2 + j]; dyl[j] = (T)0; }
#pragma unroll
                    for (int i = 0; i < D1; ++i) dxv[i] = (T)0;
                    const T w = live ? sWt[weight_offset<P>(u, v)] : (T)0;
                    const T tw = cg_backward<P>(x, y, gz, dxv, dyl);
                    if (live) {
                        if constexpr (SHARED_W) dw_acc[weight_offset<P>(u, v)] += tw;
                        else p.dW[item * (long long)W_NUMEL + weight_offset<P>(u, v)] = tw;
                    }
#pragma unroll
                    for (int i = 0; i < D1; ++i) dxl[i] = fma(w, dxv[i], dxl[i]);
                    // reduce this (instruction, v) over the warp's channels; lane 0 owns the warp's slot
#pragma unroll
                    for (int j = 0; j < D2; ++j) {
                        const T s = warp_sum(w * dyl[j]);
                        if (lane == 0) dy_slot[IN2_OFF[b] + v * D2 + j] += s;
                    }
                }
#pragma unroll
                for (int i = 0; i < D1; ++i) dxacc[C * XPC + XR_OFF[a] + i] += dxl[i];
            }
        }
    });
}

constexpr int DYREG = all_in2_mul_one() ? Y_DIM : 1;

template <int MODE>
__device__ void consumer_backward(const UvuParams& p, const Smem<true, MODE>& sm, int g, int tg) {
    using L = StageLayout<true>;
    using SM = Smem<true, MODE>;
    const int S = sm.stages;
    const int part = tg / MULG;
    const int u0 = tg % MULG;
    const int lane = tg & 31;
    const int warp = tg >> 5;
    const long long total_groups = (long long)gridDim.x * NG;
    const long long gid = (long long)blockIdx.x * NG + g;
    const long long* bnd = sm.bounds();
    const int bar_id = 1 + g;

    long long count;
    if constexpr (MODE == MODE_BATCH) {
        count = gid < p.n_items ? (p.n_items - gid + total_groups - 1) / total_groups : 0;
    } else {
        count = bnd[g + 1] - bnd[g];
    }
    const T* sWshared = reinterpret_cast<const T*>(sm.shared_w());
    unsigned char* ex = sm.extra(g);
    T* dxbuf = reinterpret_cast<T*>(ex);                           // [PS][XB/ELEM]
    T* dyslots = reinterpret_cast<T*>(ex + SM::DXBUF);             // [2][WARPS_PER_GROUP][YB/ELEM]
    T* dwacc = reinterpret_cast<T*>(ex + SM::DXBUF + SM::DYSLOT);  // [W_NUMEL] (shared weights)
    constexpr int XS = XB / ELEM, YS = YB / ELEM;

    if constexpr (SHARED_W) {
        for (int i = tg; i < W_NUMEL; i += G) dwacc[i] = (T)0;
        group_sync(bar_id, G);
    }

    T dxacc[XPC * NCH];
#pragma unroll
    for (int i = 0; i < XPC * NCH; ++i) dxacc[i] = (T)0;

    // Combine the partitions' dX partial sums through shared memory and write the row of `node`.
    auto flush = [&](long long node) {
        sfor<0, PS>([&](auto q_) {
            constexpr int Q = q_;
            if (part == Q) {
                sfor<0, NCH>([&](auto c_) {
                    constexpr int C = c_;
                    const int u = u0 + C * MULG;
                    sfor<0, N_IN1>([&](auto a_) {
                        constexpr int a = a_;
                        if constexpr (bwd_part_uses_in1(Q, a)) {
                            if ((IN1_MUL[a] == CHANNELS) || (u < IN1_MUL[a])) {
#pragma unroll
                                for (int i = 0; i < IN1_D[a]; ++i) {
                                    dxbuf[Q * XS + IN1_OFF[a] + u * IN1_D[a] + i] = dxacc[C * XPC + XR_OFF[a] + i];
                                    dxacc[C * XPC + XR_OFF[a] + i] = (T)0;
                                }
                            }
                        }
                    });
                });
            }
        });
        group_sync(bar_id, G);
        T* xrow = p.dX + node * (long long)X_DIM;
        sfor<0, N_IN1>([&](auto a_) {
            constexpr int a = a_;
            constexpr int lo = IN1_OFF[a], n = IN1_MUL[a] * IN1_D[a];
            for (int i = tg; i < n; i += G) {
                T s = (T)0;
                sfor<0, PS>([&](auto q_) {
                    constexpr int Q = q_;
                    if constexpr (bwd_part_uses_in1(Q, a)) s += dxbuf[Q * XS + lo + i];
                });
                if constexpr (MODE == MODE_ATOMIC) {
                    if constexpr (any_part_uses_in1(a)) red_add(xrow + lo + i, s);
                } else {
                    xrow[lo + i] = s;
                }
            }
        });
        group_sync(bar_id, G);
    };
    auto zero_nodes = [&](long long lo, long long hi) {
        for (long long node = lo; node < hi; ++node) {
            T* xrow = p.dX + node * (long long)X_DIM;
            for (int i = tg; i < X_DIM; i += G) xrow[i] = (T)0;
        }
    };

    long long prev = -1;
    long long next_unwritten = 0;
    if constexpr (MODE == MODE_DET) next_unwritten = bnd[NG + 1 + g];
    bool ok = true;

    for (long long it = 0; it < count; ++it) {
        const int stage = (int)(it % S);
        const long long use = it / S;
        if (!mbar_wait(sm.full(g, stage), (unsigned)(use & 1), p.status, ERR_WAIT_FULL)) {
            ok = false;
            break;
        }
        const unsigned char* st = sm.stage(g, stage);
        const long long* h = sm.hdr(g, stage);
        const long long item = h[0];
        const long long node = h[1];  // sender
        if constexpr (MODE != MODE_BATCH) {
            if (prev >= 0 && node != prev) {
                flush(prev);
                if constexpr (MODE == MODE_DET) next_unwritten = prev + 1;
            }
            if constexpr (MODE == MODE_DET) {
                if (node != prev && next_unwritten < node) zero_nodes(next_unwritten, node);
            }
            prev = node;
        }
        const T* sX = reinterpret_cast<const T*>(st + L::OFF_X);
        const T* sY = reinterpret_cast<const T*>(st + L::OFF_Y);
        const T* sWt = SHARED_W ? sWshared : reinterpret_cast<const T*>(st + L::OFF_W);
        const T* sdZ = reinterpret_cast<const T*>(st + L::OFF_DZ);
        T* slot = dyslots + ((it & 1) * WARPS_PER_GROUP + warp) * YS;
        for (int j = lane; j < Y_DIM; j += 32) slot[j] = (T)0;
        __syncwarp();

        T dyreg[DYREG];
#pragma unroll
        for (int j = 0; j < DYREG; ++j) dyreg[j] = (T)0;
        sfor<0, PS>([&](auto q_) {
            constexpr int Q = q_;
            if (part == Q) {
                sfor<0, NCH>([&](auto c_) {
                    constexpr int C = c_;
                    backward_item<Q, C>(sX, sY, sWt, sdZ, u0 + C * MULG, item, p, dwacc, slot, lane, dxacc, dyreg);
                });
            }
        });
        mbar_arrive(sm.empty(g, stage));
        if constexpr (all_in2_mul_one()) {
#pragma unroll
            for (int j = 0; j < Y_DIM; ++j) {
                const T s = warp_sum(dyreg[j]);
                if (lane == 0) slot[j] += s;
            }
        }
        if constexpr (MODE == MODE_BATCH) {
            flush(item);  // includes two group barriers, which also order the dY slots
        } else {
            group_sync(bar_id, G);
        }
        {
            const T* slots = dyslots + (it & 1) * WARPS_PER_GROUP * YS;
            for (int j = tg; j < Y_DIM; j += G) {
                T s = (T)0;
#pragma unroll
                for (int w = 0; w < WARPS_PER_GROUP; ++w) s += slots[w * YS + j];
                p.dY[item * (long long)Y_DIM + j] = s;
            }
        }
    }
    if constexpr (MODE != MODE_BATCH) {
        if (ok && prev >= 0) {
            flush(prev);
            if constexpr (MODE == MODE_DET) next_unwritten = prev + 1;
        }
        if constexpr (MODE == MODE_DET) {
            if (ok) zero_nodes(next_unwritten, bnd[NG + 2 + g]);
        }
    }
    if constexpr (SHARED_W) {
        // every (u, v, instruction) slot was accumulated by exactly one thread of the group
        group_sync(bar_id, G);
        T* out = p.ws + gid * (long long)W_NUMEL;
        for (int i = tg; i < W_NUMEL; i += G) out[i] = dwacc[i];
    }
}

// ---------------------------------------------------------------- kernel body

template <int MODE, bool BWD>
__device__ __forceinline__ void uvu_body(const UvuParams& p) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    Smem<BWD, MODE> sm(smem_raw, p.stages);
    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const bool is_producer = tid >= NCONSUMERS;

    if (tid == 0) {
        const bool any_elem = !(p.flags & 1) || !(p.flags & 2) || (!(p.flags & 4) && !SHARED_W) || (BWD && !(p.flags & 8));
        for (int g = 0; g < NG; ++g)
            for (int s = 0; s < p.stages; ++s) {
                mbar_init(sm.full(g, s), 1 + (any_elem ? 32 : 0));
                mbar_init(sm.empty(g, s), G);
            }
        fence_mbar_init();
    }
    if (is_producer) {
        if constexpr (MODE != MODE_BATCH) {
            long long* bnd = sm.bounds();
            const long long total_groups = (long long)gridDim.x * NG;
            for (int j = 0; j <= NG; ++j) {
                const long long gidx = (long long)blockIdx.x * NG + j;
                // 128-bit product not needed: n_items * groups stays far below 2^63
                const long long target = gidx >= total_groups ? p.n_items : (p.n_items / total_groups) * gidx +
                                         ((p.n_items % total_groups) * gidx) / total_groups;
                long long e = target;
                if constexpr (MODE == MODE_DET) e = align_forward<MODE, BWD>(p, target, lane);
                if (lane == 0) {
                    bnd[j] = e;
                    if constexpr (MODE == MODE_DET) {
                        long long nb = 0;
                        if (e >= p.n_items) nb = p.n_nodes;
                        else if (e > 0) nb = item_key<MODE, BWD>(p, e);
                        if (gidx == 0) nb = 0;
                        if (gidx >= total_groups) nb = p.n_nodes;
                        bnd[NG + 1 + j] = nb;
                    }
                }
            }
        }
    } else if constexpr (SHARED_W) {
        T* sw = reinterpret_cast<T*>(sm.shared_w());
        for (int i = tid; i < W_NUMEL; i += NCONSUMERS) sw[i] = p.W[i];
    }
    __syncthreads();

    if (is_producer) {
        producer<MODE, BWD>(p, sm, lane);
    } else {
        const int g = tid / G, tg = tid % G;
        if constexpr (BWD) consumer_backward<MODE>(p, sm, g, tg);
        else consumer_forward<MODE>(p, sm, g, tg);
    }
}

}  // namespace oeq

// One entry point per translation unit, selected by OEQ_KERNEL.
#define OEQ_K_FWD_BATCH 0
#define OEQ_K_BWD_BATCH 1
#define OEQ_K_FWD_DET 2
#define OEQ_K_BWD_DET 3
#define OEQ_K_FWD_ATOMIC 4
#define OEQ_K_BWD_ATOMIC 5

extern "C" __global__ void __launch_bounds__(oeq::NTHREADS, 1) oeq_uvu_kernel(const oeq::UvuParams p) {
#if OEQ_KERNEL == OEQ_K_FWD_BATCH
    oeq::uvu_body<oeq::MODE_BATCH, false>(p);
#elif OEQ_KERNEL == OEQ_K_BWD_BATCH
    oeq::uvu_body<oeq::MODE_BATCH, true>(p);
#elif OEQ_KERNEL == OEQ_K_FWD_DET
    oeq::uvu_body<oeq::MODE_DET, false>(p);
#elif OEQ_KERNEL == OEQ_K_BWD_DET
    oeq::uvu_body<oeq::MODE_DET, true>(p);
#elif OEQ_KERNEL == OEQ_K_FWD_ATOMIC
    oeq::uvu_body<oeq::MODE_ATOMIC, false>(p);
#elif OEQ_KERNEL == OEQ_K_BWD_ATOMIC
    oeq::uvu_body<oeq::MODE_ATOMIC, true>(p);
#else
#error "OEQ_KERNEL must select one of the uvu kernels"
#endif
}

// Fixed-order sum of the per-group partial weight gradients (shared weights):
// dW[i] = sum_g ws[g][i], g ascending, one thread per weight.
extern "C" __global__ void oeq_reduce_partials(const oeqd::T* ws, oeqd::T* out, int n, long long groups) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    oeqd::T s = (oeqd::T)0;
    for (long long g = 0; g < groups; ++g) s += ws[g * n + i];
    out[i] = s;
}
