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
//   * A CTA holds NG independent groups.  Each group runs its own ring of
//     shared-memory stages: its first warp stages the rows of the items ahead
//     (X gathered by sender index, Y, per-item W, and dZ gathered by receiver
//     index in the backward pass) with 1-D bulk async copies (TMA) that
//     complete on an mbarrier; rows that break the 16-byte rule fall back to
//     cp.async.  Edge indices are fetched 32 at a time, one block ahead.
//   * Work is dealt to groups in small chunks of consecutive edges, round
//     robin over all groups of the grid, so that at any moment the whole GPU
//     works on one neighbourhood of the (sorted) edge list and gathered rows
//     are re-used from L2.
//   * Clebsch-Gordan coefficients times path weights are compile-time
//     constants; the contraction is fully unrolled straight-line FMA code.
//   * Deterministic convolution: chunk boundaries are moved forward to the next
//     segment boundary (receiver runs in the forward pass, sender runs in
//     sender_perm order in the backward pass), a group accumulates a node's
//     sum in registers and writes each output row exactly once (rows without
//     edges are written as zeros), so no scratch buffer or fix-up pass exists
//     and the summation order is fixed.
//   * All waits are bounded; a wait that runs out sets *status and the group
//     stops consuming.
#pragma once
#include "oeq_common.cuh"

// kernels of this file, selected by OEQ_KERNEL
#define OEQ_K_FWD_BATCH 0
#define OEQ_K_BWD_BATCH 1
#define OEQ_K_FWD_DET 2
#define OEQ_K_BWD_DET 3
#define OEQ_K_FWD_ATOMIC 4
#define OEQ_K_BWD_ATOMIC 5
#define OEQ_K_BWD_RECV_DET 6
#define OEQ_K_BWD_RECV_ATOMIC 7
#define OEQ_K_DBL_BATCH 8
// second derivatives of the convolution: gradient with respect to dZ (forward-like walk), and the gradients with
// respect to X, Y, W (receiver-order backward-like walk)
#define OEQ_K_DBLC_Z_DET 40
#define OEQ_K_DBLC_Z_ATOMIC 41
#define OEQ_K_DBLC_G_DET 42
#define OEQ_K_DBLC_G_ATOMIC 43

namespace oeq {
using namespace oeqd;

#if defined(OEQ_KERNEL) && OEQ_KERNEL >= 40 && OEQ_KERNEL <= 43
constexpr bool DBLC = true;     // stages also carry the cotangents EX (at the sender), EY, EW
#else
constexpr bool DBLC = false;
#endif

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
    int flags;              // bit0 X bulk-able, bit1 Y, bit2 W, bit3 Z/dZ; bits 8..11: the same arrays staged by
                            // 16-byte cp.async from all lanes instead (short rows: one bulk copy per row costs
                            // the issuing lane more than the row is worth)
    int chunk;              // edges per work chunk (convolution modes)
    long long e_lo, e_hi;   // sender-row sum: the edge range [e_lo, e_hi) whose scratch rows ws holds
    // row sum done by the helper warps of a receiver-order launch (sum_items == 0: none): the whole edge list
    // in sender order, the scratch rows of the previous block and that block's edge range
    const long long* sum_cols;
    const long long* sum_perm;
    const T* sum_ws;
    long long sum_items, sum_e_lo, sum_e_hi;
    int sum_first, sum_chunk;
    // second derivatives (batch product): the cotangents of dX, dY, dW
    const T* EX;
    const T* EY;
    const T* EW;
};

constexpr int MODE_BATCH = 0;
constexpr int MODE_DET = 1;
constexpr int MODE_ATOMIC = 2;

constexpr int G = MULG * PS;
constexpr int NCONSUMERS = NG * G;
// PRODUCER = 1: one extra warp per group stages that group's items and the group's warps never meet at a
// per-item barrier (stages are handed back through "empty" mbarriers).  PRODUCER = 0: the first warp of
// each group stages that group's items itself (better when a CTA holds many small groups).
// Helper warps (deterministic receiver-order backward only): extra warps of the CTA that sum the scratch
// rows of the previous block of edges into dX while the consumers work on the current block.
#ifndef OEQ_HELPER_WARPS
#define OEQ_HELPER_WARPS 0
#endif
constexpr int HELPER_WARPS = OEQ_HELPER_WARPS;
constexpr int NSTAGING = 32 * NG * PRODUCER;                       // one staging warp per group
constexpr int NTHREADS = NCONSUMERS + NSTAGING + 32 * HELPER_WARPS;
constexpr int WARPS_PER_GROUP = G / 32;
constexpr int DY_RING = 5;   // per-item dY partials in flight; stages are capped at DY_RING - 1

// ---------------------------------------------------------------- helpers on the descriptor

__host__ __device__ constexpr int pad16(int bytes) { return (bytes + 15) / 16 * 16; }
constexpr int ELEM = sizeof(T);
constexpr int XB = pad16(X_DIM * ELEM), YB = pad16(Y_DIM * ELEM), ZB = pad16(Z_DIM * ELEM);
// UNIT_W (descriptor): the problem has no weight array, every weight is 1 (the product summed per receiver
// before a shared dense contraction): nothing is staged for W and no weight gradient is written.
constexpr int WB = (SHARED_W || UNIT_W) ? 0 : pad16(W_NUMEL * ELEM);
constexpr int SWB = SHARED_W ? pad16(W_NUMEL * ELEM) : 0;

// Backward staging in phases: with NPH > 1 an edge is staged as NPH items.  Phase q carries the weights
// [W_PH_BEGIN[q], W_PH_BEGIN[q+1]) and the output-gradient columns [Z_PH_BEGIN[q], Z_PH_BEGIN[q+1]) of
// the instructions assigned to it; X and Y travel with phase 0.  A stage then holds only a slice of the
// (large) output-gradient row, so several groups fit per SM.
constexpr int NPH = BWD_NPH;
constexpr int imax(int a, int b) { return a > b ? a : b; }
constexpr int max_phase_width(const int* begin) {
    int m = 0;
    for (int q = 0; q < NPH; ++q) m = imax(m, begin[q + 1] - begin[q]);
    return m;
}
constexpr int WPHB = (SHARED_W || UNIT_W) ? 0 : pad16(max_phase_width(W_PH_BEGIN) * ELEM);
constexpr int ZPHB = pad16(max_phase_width(Z_PH_BEGIN) * ELEM);

// Edges per staged item (descriptor constant EPI).  Narrow problems (a group is one warp) spend more instructions on
// walking the edge list, issuing copies and barrier hand-offs than on arithmetic; with EPI > 1 an item is up to EPI
// consecutive edges of the receiver-ordered list: one hand-off, one header, one copy of their Y rows and one of their
// W rows (consecutive edges are contiguous there; rows unpadded), EPI gathered X rows.  Only the walks in
// receiver order (forward pass, receiver-order backward pass) without staging warps use it.
constexpr int HDR_SLOTS = EPI > 1 ? 4 + 2 * EPI : 4;     // edge/count, node bounds; then receivers and senders
constexpr int SLOT_BYTES = 16 + 8 * HDR_SLOTS;           // two barriers and the header per (group, stage)
constexpr int YBK = EPI > 1 ? pad16(EPI * Y_DIM * ELEM) : YB;
constexpr int WBK = EPI > 1 ? ((SHARED_W || UNIT_W) ? 0 : pad16(EPI * W_NUMEL * ELEM)) : WB;

template <bool BWD>
struct StageLayout {
    static constexpr int OFF_X = 0;
    static constexpr int OFF_Y = OFF_X + (BWD ? 1 : EPI) * XB;
    static constexpr int OFF_W = OFF_Y + (BWD ? YB : YBK);
    static constexpr int OFF_DZ = OFF_W + (BWD ? WPHB : WBK);
    static constexpr int OFF_EX = OFF_DZ + (BWD ? ZPHB : 0);       // cotangent rows (second derivatives of the
    static constexpr int OFF_EY = OFF_EX + (DBLC ? XB : 0);        // convolution only)
    static constexpr int OFF_EW = OFF_EY + (DBLC ? YB : 0);
    static constexpr int BYTES = OFF_EW + (DBLC ? WB : 0);
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
constexpr bool fwd_part_uses_in2(int q, int b) {
    for (int p = 0; p < N_INSTR; ++p)
        if (FWD_PART_OF_OUT[I_OUT[p]] == q && I_IN2[p] == b) return true;
    return false;
}
constexpr bool bwd_part_uses_in2(int q, int b) {
    for (int p = 0; p < N_INSTR; ++p)
        if (BWD_PART_OF_INSTR[p] == q && I_IN2[p] == b) return true;
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
constexpr int next_pow2(int n) {
    int p = 1;
    while (p < n) p *= 2;
    return p;
}
constexpr int CHANNELS = MULG * NCH;
// second-input rows are kept in registers when every multiplicity is 1 and the row is short
constexpr bool Y_IN_REGS = all_in2_mul_one() && Y_DIM <= 32;

// Same (i, j) pair as the previous / next Clebsch-Gordan entry of the same instruction?
template <int P, int N>
constexpr bool cg_pair_first() {
    return N == CG_BEGIN[P] || CG_I[N] != CG_I[N - 1] || CG_J[N] != CG_J[N - 1];
}
template <int P, int N>
constexpr bool cg_pair_last() {
    return N == CG_BEGIN[P + 1] - 1 || CG_I[N] != CG_I[N + 1] || CG_J[N] != CG_J[N + 1];
}

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

// t[k] += sum_n c_n * (x[i_n] * y[j_n]); the product of a pair is formed once.
template <int P, class XA, class YA, class TA>
__device__ __forceinline__ void cg_forward(const XA& x, const YA& y, TA& t) {
    T xy = (T)0;
    sfor<CG_BEGIN[P], CG_BEGIN[P + 1]>([&](auto n) {
        constexpr int N = n;
        if constexpr (cg_pair_first<P, N>()) xy = x[CG_I[N]] * y[CG_J[N]];
        t[CG_K[N]] = fma(xy, (T)CG_V[N], t[CG_K[N]]);
    });
}

// Backward of the above for one (u, v) with g = dZ block of the channel:
//   P_ij = sum_k c_ijk g_k;  a_i += y_j P_ij;  b_j += x_i P_ij
// so that dX_i = w a_i, dY_j = w b_j and dW = sum_i x_i a_i.
template <int P, class XA, class YA, class GA, class AA, class BA>
__device__ __forceinline__ void cg_backward(const XA& x, const YA& y, const GA& g, AA& a, BA& b) {
    T pij = (T)0;
    sfor<CG_BEGIN[P], CG_BEGIN[P + 1]>([&](auto n) {
        constexpr int N = n;
        if constexpr (cg_pair_first<P, N>()) pij = (T)CG_V[N] * g[CG_K[N]];
        else pij = fma((T)CG_V[N], g[CG_K[N]], pij);
        if constexpr (cg_pair_last<P, N>()) {
            a[CG_I[N]] = fma(y[CG_J[N]], pij, a[CG_I[N]]);
            b[CG_J[N]] = fma(x[CG_I[N]], pij, b[CG_J[N]]);
        }
    });
}

// Second-derivative form of the above (convolution): with r = w ex + ew x,
//   ay_i += y_j P_ij;  aey_i += ey_j P_ij;  b_j += r_i P_ij.
template <int P, class RA, class YA, class EA, class GA, class AA, class BA>
__device__ __forceinline__ void cg_backward_dbl(const RA& r, const YA& y, const EA& ey, const GA& g, AA& ay, AA& aey, BA& b) {
    T pij = (T)0;
    sfor<CG_BEGIN[P], CG_BEGIN[P + 1]>([&](auto n) {
        constexpr int N = n;
        if constexpr (cg_pair_first<P, N>()) pij = (T)CG_V[N] * g[CG_K[N]];
        else pij = fma((T)CG_V[N], g[CG_K[N]], pij);
        if constexpr (cg_pair_last<P, N>()) {
            ay[CG_I[N]] = fma(y[CG_J[N]], pij, ay[CG_I[N]]);
            aey[CG_I[N]] = fma(ey[CG_J[N]], pij, aey[CG_I[N]]);
            b[CG_J[N]] = fma(r[CG_I[N]], pij, b[CG_J[N]]);
        }
    });
}

// Sum each of v[0..N) over the 32 lanes in a fixed order with N + log-many shuffles
// (recursive halving); afterwards lane L holds the total of index L >> (5 - log2(NP)) in v[0].
template <int N, class VA>
__device__ __forceinline__ void warp_reduce_vector(VA& v, int lane) {
    constexpr int NP = next_pow2(N);
    T w[NP];
#pragma unroll
    for (int i = 0; i < NP; ++i) w[i] = i < N ? v[i] : (T)0;
    int count = NP;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        if (count > 1) {
            const int half = count / 2;
            const bool upper = (lane & off) != 0;
#pragma unroll
            for (int m = 0; m < NP / 2; ++m) {
                if (m < half) {
                    const T send = upper ? w[m] : w[m + half];
                    const T keep = upper ? w[m + half] : w[m];
                    w[m] = keep + __shfl_xor_sync(0xffffffffu, send, off);
                }
            }
            count = half;
        } else {
            w[0] += __shfl_xor_sync(0xffffffffu, w[0], off);
        }
    }
    v[0] = w[0];
}
constexpr int log2_int(int n) {
    int l = 0;
    while ((1 << l) < n) ++l;
    return l;
}

// ---------------------------------------------------------------- shared memory map

// RECV: the receiver-order backward pass of the convolution.  It stages what the forward pass stages
// (X of the sender, Y, W of the edge) and keeps two per-edge dX rows and the dY partials as extras.
template <bool BWD, int MODE, bool RECV = false>
struct Smem {
    using L = StageLayout<BWD && !RECV>;
    // per-group extras
    static constexpr int ZBUF = (!BWD && MODE == MODE_BATCH) ? 2 * ZB : 0;      // staged output rows
    static constexpr int DXBUF = BWD ? (RECV ? 2 * XB : PS * XB) : 0;           // dX partials per partition / two dX rows
    static constexpr int DYSLOT = BWD ? DY_RING * WARPS_PER_GROUP * YB : 0;     // per-warp dY partials, a ring over items
    static constexpr int DWACC = (BWD && SHARED_W) ? pad16(W_NUMEL * ELEM) : 0; // shared-weight gradient
    static constexpr int GZS = RECV ? pad16(GZ_SMEM_VALUES * G * ELEM) : 0;     // parked dZ values (receiver order)
    static constexpr int EXTRA = ZBUF + DXBUF + DYSLOT + DWACC + GZS;

    unsigned char* base;
    int stages;
    __device__ Smem(unsigned char* b, int s) : base(b), stages(s) {}
    static constexpr int CTRL = 128;   // per group: item count (8 B), then DY_RING arrival counters at +16
    __device__ unsigned long long* full(int g, int s) const {
        return reinterpret_cast<unsigned long long*>(base) + (g * stages + s) * 2;
    }
    __device__ unsigned long long* empty(int g, int s) const { return full(g, s) + 1; }
    __device__ long long* hdr(int g, int s) const {
        return reinterpret_cast<long long*>(base + NG * stages * 16) + (g * stages + s) * HDR_SLOTS;
    }
    __device__ long long* total(int g) const {   // number of items of the group, -1 until known
        return reinterpret_cast<long long*>(base + NG * stages * SLOT_BYTES + g * CTRL);
    }
    __device__ int* arrivals(int g) const { return reinterpret_cast<int*>(base + NG * stages * SLOT_BYTES + g * CTRL + 16); }
    __device__ unsigned char* shared_w() const { return base + NG * stages * SLOT_BYTES + NG * CTRL; }
    __device__ unsigned char* group_base(int g) const {
        return shared_w() + SWB + (long long)g * (stages * L::BYTES + EXTRA);
    }
    __device__ unsigned char* stage(int g, int s) const { return group_base(g) + s * L::BYTES; }
    __device__ unsigned char* extra(int g) const { return group_base(g) + stages * L::BYTES; }
};

// ---------------------------------------------------------------- work assignment and staging

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

// The sequence of items of one group, walked by the group's first warp (all 32 lanes in step).
// Batch mode: rows gid, gid + groups, ...  Convolution modes: chunks gid, gid + groups, ... of
// `chunk` consecutive edges each (deterministic: chunk ends moved to segment boundaries).
template <int MODE, bool BWD>
struct ItemWalker {
    const UvuParams& p;
    long long groups, gid;
    int lane;
    // batch
    long long next_row;
    // convolution: current chunk [pos, end), chunk index, node range of the chunk
    long long chunk_index, pos, end, node_lo, node_hi, n_chunks;
    bool first_in_chunk;
    // indices of up to 32 items starting at block_base, one per lane
    long long block_base, ie, is_, ir;

    __device__ ItemWalker(const UvuParams& p_, long long groups_, long long gid_, int lane_)
        : p(p_), groups(groups_), gid(gid_), lane(lane_) {
        next_row = gid;
        n_chunks = (p.n_items + p.chunk - 1) / p.chunk;
        chunk_index = gid - groups;
        pos = end = 0;
        node_lo = node_hi = 0;
        first_in_chunk = false;
        block_base = -1;
        ie = is_ = ir = 0;
    }

    __device__ long long chunk_start(long long c) const {
        const long long t = c * p.chunk;
        if constexpr (MODE == MODE_DET) return align_forward<MODE, BWD>(p, t, lane);
        return t < p.n_items ? t : p.n_items;
    }
    __device__ long long node_bound(long long c, long long e) const {
        if (c <= 0) return 0;
        if (e >= p.n_items) return p.n_nodes;
        return item_key<MODE, BWD>(p, e);
    }

    // Advance to the next non-empty chunk; false when the group's work is exhausted.
    __device__ bool next_chunk() {
        for (;;) {
            chunk_index += groups;
            if (chunk_index >= n_chunks) return false;
            pos = chunk_start(chunk_index);
            end = chunk_index + 1 >= n_chunks ? p.n_items : chunk_start(chunk_index + 1);
            if constexpr (MODE == MODE_DET) {
                node_lo = node_bound(chunk_index, pos);
                node_hi = chunk_index + 1 >= n_chunks ? p.n_nodes : node_bound(chunk_index + 1, end);
            }
            if (end > pos) {
                first_in_chunk = true;
                block_base = -1;
                return true;
            }
        }
    }

    // Next run of up to EPI consecutive edges of the chunk (receiver-order walks): first edge e0, count, and in
    // lane i < count the sender and receiver of edge e0 + i.  A run ends at a multiple of EPI (so that full runs
    // start 16-byte aligned in the per-edge arrays), at the chunk's end or at the end of the 32-edge window.
    __device__ bool next_block(long long& e0, int& cnt, long long& s_i, long long& r_i, long long& lo, long long& hi) {
        static_assert(!(BWD && MODE == MODE_DET) || EPI == 1, "runs of edges need the list's own order");
        lo = hi = -1;
        if (pos >= end) {
            if (!next_chunk()) return false;
        }
        if (block_base < 0 || pos >= block_base + 32) {
            block_base = pos;
            const long long k = pos + lane;
            long long ls = 0, lr = 0;
            if (k < end) {
                ls = p.cols[k];
                lr = p.rows[k];
            }
            is_ = ls; ir = lr;
        }
        const int src = (int)(pos - block_base);
        long long n = end - pos;
        const long long to_boundary = EPI - (pos % EPI);
        if (to_boundary < n) n = to_boundary;
        if (32 - src < n) n = 32 - src;
        cnt = (int)n;
        e0 = pos;
        s_i = __shfl_sync(0xffffffffu, is_, (src + lane) & 31);
        r_i = __shfl_sync(0xffffffffu, ir, (src + lane) & 31);
        if (first_in_chunk) {
            lo = node_lo;
            first_in_chunk = false;
        }
        pos += cnt;
        if (pos >= end) hi = node_hi;
        return true;
    }

    // Next item: edge/row index e, sender s, receiver r, and the chunk's node range when the
    // item opens (lo >= 0) or closes (hi >= 0) a chunk.  Returns false at the end.
    __device__ bool next(long long& e, long long& s, long long& r, long long& lo, long long& hi) {
        lo = hi = -1;
        if constexpr (MODE == MODE_BATCH) {
            if (next_row >= p.n_items) return false;
            e = s = r = next_row;
            next_row += groups;
            return true;
        } else {
            if (pos >= end) {
                if (!next_chunk()) return false;
            }
            if (block_base < 0 || pos >= block_base + 32) {
                block_base = pos;
                const long long k = pos + lane;
                long long le = 0, ls = 0, lr = 0;
                if (k < end) {
                    le = (BWD && MODE == MODE_DET) ? p.perm[k] : k;
                    ls = p.cols[le];
                    lr = p.rows[le];
                }
                ie = le; is_ = ls; ir = lr;
            }
            const int src = (int)(pos - block_base);
            e = __shfl_sync(0xffffffffu, ie, src);
            s = __shfl_sync(0xffffffffu, is_, src);
            r = __shfl_sync(0xffffffffu, ir, src);
            if (first_in_chunk) {
                lo = node_lo;
                first_in_chunk = false;
            }
            ++pos;
            if (pos >= end) hi = node_hi;
            return true;
        }
    }
};

// Stage one item into ring slot `stage` (executed by the group's first warp).
template <int MODE, bool BWD, class SMT>
__device__ __forceinline__ void issue_item(const UvuParams& p, const SMT& sm, int g, int stage, int lane,
                                           long long e, long long s, long long r, long long lo, long long hi,
                                           int ph = 0) {
    using L = StageLayout<BWD>;
    const bool first = ph == 0;                       // X and Y travel with the first phase only
    const bool xb = p.flags & 1, yb = p.flags & 2, wb = p.flags & 4, zb = p.flags & 8;
    unsigned char* st = sm.stage(g, stage);
    unsigned long long* full = sm.full(g, stage);
    const T* xsrc = p.X + s * X_DIM;
    const T* ysrc = p.Y + e * Y_DIM;
    // weights and output gradient: the whole row, or this phase's part of it
    const int w_lo = BWD ? W_PH_BEGIN_DEV[ph] : 0, w_n = BWD ? W_PH_BEGIN_DEV[ph + 1] - w_lo : W_NUMEL;
    const int z_lo = BWD ? Z_PH_BEGIN_DEV[ph] : 0, z_n = BWD ? Z_PH_BEGIN_DEV[ph + 1] - z_lo : Z_DIM;
    const T* wsrc = (SHARED_W || UNIT_W) ? nullptr : p.W + e * (long long)W_NUMEL + w_lo;
    const T* zsrc = BWD ? p.dZ + r * (long long)Z_DIM + z_lo : nullptr;
    const unsigned wbytes = (unsigned)pad16(w_n * ELEM), zbytes = (unsigned)pad16(z_n * ELEM);
    if (lane == 0) {
        long long* h = sm.hdr(g, stage);
        h[0] = e;
        h[1] = BWD ? s : r;
        h[2] = lo;
        h[3] = hi;
        unsigned bytes = 0;
        if (xb && first) bytes += XB;
        if (yb && first) bytes += YB;
        if (wb && !SHARED_W) bytes += wbytes;
        if (BWD && zb) bytes += zbytes;
        if constexpr (DBLC) bytes += (xb ? XB : 0) + (yb ? YB : 0) + (wb ? WB : 0);
        mbar_arrive_expect_tx(full, bytes);
        if constexpr (DBLC) {
            if (xb) bulk_g2s(st + L::OFF_EX, p.EX + s * X_DIM, XB, full);
            if (yb) bulk_g2s(st + L::OFF_EY, p.EY + e * Y_DIM, YB, full);
            if (wb) bulk_g2s(st + L::OFF_EW, p.EW + e * (long long)W_NUMEL, WB, full);
        }
        if constexpr (MODE == MODE_BATCH) {
            if (BWD && zb) bulk_g2s(st + L::OFF_DZ, zsrc, zbytes, full);
            if (wb && !SHARED_W) bulk_g2s(st + L::OFF_W, wsrc, wbytes, full);
            if (xb && first) bulk_g2s(st + L::OFF_X, xsrc, XB, full);
            if (yb && first) bulk_g2s(st + L::OFF_Y, ysrc, YB, full);
        } else {
            // gathered node rows are needed again by neighbouring edges; per-edge rows are read once
            const unsigned long long keep = l2_policy_evict_last(), stream = l2_policy_evict_first();
            if (BWD && zb) bulk_g2s_hint(st + L::OFF_DZ, zsrc, zbytes, full, keep);
            if (wb && !SHARED_W) bulk_g2s_hint(st + L::OFF_W, wsrc, wbytes, full, stream);
            if (xb && first) bulk_g2s_hint(st + L::OFF_X, xsrc, XB, full, keep);
            if (yb && first) bulk_g2s_hint(st + L::OFF_Y, ysrc, YB, full, stream);
        }
    }
    const bool any_elem = !xb || !yb || (!wb && !SHARED_W && !UNIT_W) || (BWD && !zb);
    if (any_elem) {
        // rows that are not bulk copied: 16-byte pieces by all lanes when the row allows it, single elements otherwise
        auto stage_row = [&](unsigned char* dst, const T* src, int n, bool vec) {
            if (vec) {
                const int pieces = pad16(n * ELEM) / 16;
                for (int i = lane; i < pieces; i += 32) cp_async_16(dst + 16 * i, reinterpret_cast<const unsigned char*>(src) + 16 * i);
            } else {
                for (int i = lane; i < n; i += 32) cp_async_elem<ELEM>((T*)dst + i, src + i);
            }
        };
        if (!xb && first) stage_row(st + L::OFF_X, xsrc, X_DIM, p.flags & 256);
        if (!yb && first) stage_row(st + L::OFF_Y, ysrc, Y_DIM, p.flags & 512);
        if constexpr (!SHARED_W && !UNIT_W) {
            if (!wb) stage_row(st + L::OFF_W, wsrc, w_n, p.flags & 1024);
        }
        if constexpr (BWD) {
            if (!zb) stage_row(st + L::OFF_DZ, zsrc, z_n, p.flags & 2048);
        }
        if constexpr (DBLC) {
            if (!xb) stage_row(st + L::OFF_EX, p.EX + s * X_DIM, X_DIM, false);
            if (!yb) stage_row(st + L::OFF_EY, p.EY + e * Y_DIM, Y_DIM, false);
            if (!wb) stage_row(st + L::OFF_EW, p.EW + e * (long long)W_NUMEL, W_NUMEL, false);
        }
        cp_async_arrive_noinc(full);
    }
}

// Stage a run of `cnt` consecutive edges starting at e0 into ring slot `stage` (EPI > 1; all lanes of the
// group's first warp; lane i < cnt holds sender and receiver of edge e0 + i).  Header: e0, cnt, lo, hi, then the
// receivers, then the senders.  The barrier always takes the 32 per-lane arrivals (rows of a short run may
// not qualify for a bulk copy).
template <int MODE, class SMT>
__device__ __forceinline__ void issue_block(const UvuParams& p, const SMT& sm, int g, int stage, int lane,
                                            long long e0, int cnt, long long s_i, long long r_i, long long lo, long long hi) {
    using L = StageLayout<false>;
    const bool xb = p.flags & 1, yb = p.flags & 2, wb = p.flags & 4;
    unsigned char* st = sm.stage(g, stage);
    unsigned long long* full = sm.full(g, stage);
    long long* h = sm.hdr(g, stage);
    const unsigned ybytes = (unsigned)(cnt * Y_DIM * ELEM), wbytes = (unsigned)(cnt * W_NUMEL * ELEM);
    const bool y_bulk = yb && (ybytes % 16u) == 0;
    const bool w_bulk = !SHARED_W && !UNIT_W && wb && (wbytes % 16u) == 0;
    const T* ysrc = p.Y + e0 * Y_DIM;
    const T* wsrc = (SHARED_W || UNIT_W) ? nullptr : p.W + e0 * (long long)W_NUMEL;
    if (lane < cnt) {
        h[4 + lane] = r_i;
        h[4 + EPI + lane] = s_i;
    }
    if (lane == 0) {
        h[0] = e0;
        h[1] = cnt;
        h[2] = lo;
        h[3] = hi;
    }
    __syncwarp();       // the header is complete before lane 0's arrival publishes it
    const unsigned long long keep = l2_policy_evict_last(), stream = l2_policy_evict_first();
    if (lane == 0) {
        mbar_arrive_expect_tx(full, (xb ? (unsigned)cnt * XB : 0u) + (y_bulk ? ybytes : 0u) + (w_bulk ? wbytes : 0u));
        if (w_bulk) bulk_g2s_hint(st + L::OFF_W, wsrc, wbytes, full, stream);
        if (y_bulk) bulk_g2s_hint(st + L::OFF_Y, ysrc, ybytes, full, stream);
    }
    __syncwarp();       // the byte count is posted before any lane's copy can complete
    if (xb && lane < cnt) bulk_g2s_hint(st + L::OFF_X + lane * XB, p.X + s_i * X_DIM, XB, full, keep);
    if (!xb) {
        for (int i = 0; i < cnt; ++i) {
            const long long s = __shfl_sync(0xffffffffu, s_i, i);
            for (int q = lane; q < X_DIM; q += 32) cp_async_elem<ELEM>((T*)(st + L::OFF_X + i * XB) + q, p.X + s * X_DIM + q);
        }
    }
    if (!y_bulk)
        for (int q = lane; q < cnt * Y_DIM; q += 32) cp_async_elem<ELEM>((T*)(st + L::OFF_Y) + q, ysrc + q);
    if constexpr (!SHARED_W && !UNIT_W) {
        if (!w_bulk)
            for (int q = lane; q < cnt * W_NUMEL; q += 32) cp_async_elem<ELEM>((T*)(st + L::OFF_W) + q, wsrc + q);
    }
    cp_async_arrive_noinc(full);
}

// Producer warp of group g: stages the group's items as stage slots are handed back.
// SENDER_IN_HEADER: header slot 2 carries the edge's sender instead of the chunk's first node (the
// receiver-order backward pass needs both end points of an edge and no node bounds).
template <int MODE, bool BWD, bool SENDER_IN_HEADER = false, class SMT>
__device__ void run_producer(const UvuParams& p, const SMT& sm, int g, int lane) {
    const int S = sm.stages;
    ItemWalker<MODE, BWD> walker(p, (long long)gridDim.x * NG, (long long)blockIdx.x * NG + g, lane);
    constexpr int PHASES = BWD ? NPH : 1;
    volatile long long* total = sm.total(g);
    long long it = 0;
    bool ok = true;
    // optional cycle accounting (flags bit 4: p.ws is a counter buffer): producer of CTA 0's first group
    const bool prof = UVU_PROFILE && BWD && !SHARED_W && (p.flags & 16) && blockIdx.x == 0 && g == 0 && lane == 0;
    unsigned long long prof_wait = 0, prof_walk = 0, prof_issue = 0;
    const long long prof_begin = prof ? clock64() : 0;
    while (ok) {
        long long e, s, r, lo, hi;
        const long long tw = prof ? clock64() : 0;
        const bool got = walker.next(e, s, r, lo, hi);
        if (prof) prof_walk += (unsigned long long)(clock64() - tw);
        if (!got) break;
        for (int ph = 0; ph < PHASES && ok; ++ph, ++it) {
            const int stage = (int)(it % S);
            const long long t0 = prof ? clock64() : 0;
            if (it >= S) ok = mbar_wait(sm.empty(g, stage), (unsigned)(((it / S) - 1) & 1), p.status, ERR_WAIT_EMPTY);
            const long long t1 = prof ? clock64() : 0;
            if (ok) issue_item<MODE, BWD>(p, sm, g, stage, lane, e, s, r, SENDER_IN_HEADER ? s : lo, hi, ph);
            if (prof) {
                prof_wait += (unsigned long long)(t1 - t0);
                prof_issue += (unsigned long long)(clock64() - t1);
            }
        }
    }
    if (prof) {
        unsigned long long* out = reinterpret_cast<unsigned long long*>(p.ws);
        out[4] = (unsigned long long)(clock64() - prof_begin);   // producer: total cycles
        out[5] = prof_wait;                                      // ... of which waiting for a free stage,
        out[6] = prof_walk;                                      // walking the edge list,
        out[7] = prof_issue;                                     // issuing the copies
    }
    if (lane == 0) *total = it - (ok ? 0 : 1);
    asm volatile("cp.async.wait_all;" ::: "memory");
}

// Wait until item `it` of group g has landed.  0: landed, 1: the group has no such item, 2: gave up.
template <int MODE, bool BWD, class SMT>
__device__ __forceinline__ int acquire_item(const UvuParams& p, const SMT& sm, int g, long long it) {
    const int S = sm.stages;
    const int stage = (int)(it % S);
    volatile long long* total = sm.total(g);
    if constexpr (!PRODUCER) {
        // the staging warp runs S - 1 items ahead, so the count (once written) is already visible through
        // the barrier that ended the previous iteration
        const long long n = *total;
        if (n >= 0 && it >= n) return 1;
        return mbar_wait(sm.full(g, stage), (unsigned)((it / S) & 1), p.status, ERR_WAIT_FULL) ? 0 : 2;
    } else {
        for (unsigned spin = 0; spin < WAIT_LIMIT; ++spin) {
            if (mbar_try_wait(sm.full(g, stage), (unsigned)((it / S) & 1))) return 0;
            const long long n = *total;
            if (n >= 0 && it >= n) return 1;
        }
        if (p.status) atomicCAS(p.status, 0, ERR_WAIT_FULL);
        return 2;
    }
}

// Hand stage `stage` back to the producer warp (PRODUCER mode): one arrival per consumer warp.
template <int MODE, bool BWD, class SMT>
__device__ __forceinline__ void release_stage(const SMT& sm, int g, int stage, int lane) {
    __syncwarp();
    if (lane == 0) mbar_arrive(sm.empty(g, stage));
}

// ---------------------------------------------------------------- forward

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
    T yr[Y_IN_REGS ? Y_DIM : 1];
    if constexpr (Y_IN_REGS) {
        sfor<0, N_IN2>([&](auto b_) {
            constexpr int b = b_;
            if constexpr (fwd_part_uses_in2(Q, b)) {
#pragma unroll
                for (int j = 0; j < IN2_D[b]; ++j) yr[IN2_OFF[b] + j] = sY[IN2_OFF[b] + j];
            }
        });
    }
    sfor<0, N_OUT>([&](auto o_) {
        constexpr int o = o_;
        if constexpr (FWD_PART_OF_OUT[o] == Q) {
            constexpr int D3 = OUT_D[o];
            sfor<0, N_INSTR>([&](auto p_) {
                constexpr int P = p_;
                if constexpr (I_OUT[P] == o) {
                    constexpr int a = I_IN1[P], b = I_IN2[P];
                    constexpr int D2 = IN2_D[b], M2 = IN2_MUL[b];
                    if ((IN1_MUL[a] == CHANNELS) || (u < IN1_MUL[a])) {
                        const T* x = xr + XR_OFF[a];
                        if constexpr (M2 == 1) {
                            T t[D3];
#pragma unroll
                            for (int k = 0; k < D3; ++k) t[k] = (T)0;
                            if constexpr (Y_IN_REGS) {
                                cg_forward<P>(x, yr + IN2_OFF[b], t);
                            } else {
                                T y[D2];
#pragma unroll
                                for (int j = 0; j < D2; ++j) y[j] = sY[IN2_OFF[b] + j];
                                cg_forward<P>(x, y, t);
                            }
                            const T w = UNIT_W ? (T)1 : sWt[weight_offset<P>(u, 0)];
#pragma unroll
                            for (int k = 0; k < D3; ++k)
                                zacc[C * ZPC_MAX + ZR_OFF[o] + k] = fma(w, t[k], zacc[C * ZPC_MAX + ZR_OFF[o] + k]);
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
                                const T w = UNIT_W ? (T)1 : sWt[weight_offset<P>(u, v)];
#pragma unroll
                                for (int k = 0; k < D3; ++k)
                                    zacc[C * ZPC_MAX + ZR_OFF[o] + k] = fma(w, t[k], zacc[C * ZPC_MAX + ZR_OFF[o] + k]);
                            }
                        }
                    }
                }
            });
        }
    });
}

// Forward-like pass of the convolution's second derivatives: this edge's contribution to the gradient with
// respect to dZ, T(ex, y, w) + T(x, ey, w) + T(x, y, ew), as one contraction: with r_i = w ex_i + ew x_i,
//   t_ij = r_i y_j + (w x_i) ey_j,   z_k += C_ijk t_ij.
template <class ZA>
__device__ __forceinline__ void forward_item_dbl(const T* __restrict__ sX, const T* __restrict__ sEX,
                                                 const T* __restrict__ sY, const T* __restrict__ sEY,
                                                 const T* __restrict__ sW, const T* __restrict__ sEW, int u, ZA& zacc) {
    T yr[Y_DIM], eyr[Y_DIM];
#pragma unroll
    for (int j = 0; j < Y_DIM; ++j) { yr[j] = sY[j]; eyr[j] = sEY[j]; }
    sfor<0, N_IN1>([&](auto a_) {
        constexpr int a = a_;
        constexpr int D1 = IN1_D[a];
        const bool live = (IN1_MUL[a] == CHANNELS) || (u < IN1_MUL[a]);
        T x[D1], ex[D1];
#pragma unroll
        for (int i = 0; i < D1; ++i) {
            x[i] = live ? sX[IN1_OFF[a] + u * D1 + i] : (T)0;
            ex[i] = live ? sEX[IN1_OFF[a] + u * D1 + i] : (T)0;
        }
        sfor<0, N_INSTR>([&](auto p_) {
            constexpr int P = p_;
            if constexpr (I_IN1[P] == a) {
                constexpr int b = I_IN2[P], o = I_OUT[P];
                const T w = live ? sW[weight_offset<P>(u, 0)] : (T)0;
                const T ew = live ? sEW[weight_offset<P>(u, 0)] : (T)0;
                T r[D1], wx[D1];
#pragma unroll
                for (int i = 0; i < D1; ++i) { r[i] = fma(w, ex[i], ew * x[i]); wx[i] = w * x[i]; }
                T tij = (T)0;
                sfor<CG_BEGIN[P], CG_BEGIN[P + 1]>([&](auto n) {
                    constexpr int N = n;
                    if constexpr (cg_pair_first<P, N>())
                        tij = fma(r[CG_I[N]], yr[IN2_OFF[b] + CG_J[N]], wx[CG_I[N]] * eyr[IN2_OFF[b] + CG_J[N]]);
                    zacc[ZR_OFF[o] + CG_K[N]] = fma((T)CG_V[N], tij, zacc[ZR_OFF[o] + CG_K[N]]);
                });
            }
        });
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
__device__ void run_forward(const UvuParams& p, const Smem<false, MODE>& sm, int g, int tg) {
    using L = StageLayout<false>;
    const int S = sm.stages;
    const int part = tg / MULG;
    const int u0 = tg % MULG;
    const int lane = tg & 31;
    const bool issuer = tg < 32;
    const long long total_groups = (long long)gridDim.x * NG;
    const long long gid = (long long)blockIdx.x * NG + g;
    const int bar_id = 1 + g;

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

    // without a producer warp the group's first warp walks the item sequence S - 1 items ahead
    ItemWalker<MODE, false> walker(p, total_groups, gid, lane);
    long long issued = 0;
    bool more = true;
    auto issue_next = [&]() {
        if (!more) return;
        if constexpr (EPI > 1) {
            static_assert(EPI == 1 || (!PRODUCER && MODE != MODE_BATCH && !DBLC), "runs of edges: self-staging convolution walks");
            long long e0, s_i, r_i, lo, hi;
            int cnt;
            more = walker.next_block(e0, cnt, s_i, r_i, lo, hi);
            if (more) {
                issue_block<MODE>(p, sm, g, (int)(issued % S), lane, e0, cnt, s_i, r_i, lo, hi);
                ++issued;
            } else if (lane == 0) {
                *reinterpret_cast<volatile long long*>(sm.total(g)) = issued;
            }
        } else {
            long long e, s, r, lo, hi;
            more = walker.next(e, s, r, lo, hi);
            if (more) {
                issue_item<MODE, false>(p, sm, g, (int)(issued % S), lane, e, s, r, lo, hi);
                ++issued;
            } else if (lane == 0) {
                *reinterpret_cast<volatile long long*>(sm.total(g)) = issued;
            }
        }
    };
    if constexpr (!PRODUCER) {
        if (issuer) {
            for (int i = 0; i < S - 1; ++i) issue_next();
        }
        group_sync(bar_id, G);
    }

    long long prev = -1;
    long long next_unwritten = 0;
    for (long long it = 0;; ++it) {
        const int stage = (int)(it % S);
        if constexpr (!PRODUCER) {
            // stage (it + S - 1) % S was released by the barrier that ended the previous iteration
            if (issuer) issue_next();
        }
        if (acquire_item<MODE, false>(p, sm, g, it) != 0) break;
        const long long* h = sm.hdr(g, stage);
        const unsigned char* st = sm.stage(g, stage);
        const int n_edges = EPI > 1 ? (int)h[1] : 1;
        for (int ei = 0; ei < n_edges; ++ei) {       // the edges of the item (one unless EPI > 1)
            const long long node = EPI > 1 ? h[4 + ei] : h[1];
            const long long lo = (EPI == 1 || ei == 0) ? h[2] : -1;
            const long long hi = (EPI == 1 || ei == n_edges - 1) ? h[3] : -1;
            if constexpr (MODE != MODE_BATCH) {
                if (lo >= 0) next_unwritten = lo;   // a new chunk starts: its first node is unwritten
                if (prev >= 0 && node != prev) {
                    flush(prev);
                    if constexpr (MODE == MODE_DET) next_unwritten = prev + 1 > next_unwritten ? prev + 1 : next_unwritten;
                }
                if constexpr (MODE == MODE_DET) {
                    if (next_unwritten < node) zero_nodes(next_unwritten, node);
                    next_unwritten = node + 1;
                }
                prev = node;
            }
            const T* sX = reinterpret_cast<const T*>(st + L::OFF_X + (EPI > 1 ? ei * XB : 0));
            const T* sY = reinterpret_cast<const T*>(st + L::OFF_Y) + (EPI > 1 ? ei * Y_DIM : 0);
            const T* sWt = SHARED_W ? sWshared : reinterpret_cast<const T*>(st + L::OFF_W) + (EPI > 1 ? ei * W_NUMEL : 0);
            if constexpr (DBLC) {
                static_assert(!DBLC || (PS == 1 && NCH == 1 && Y_IN_REGS && !SHARED_W && !UNIT_W), "one thread per channel");
                forward_item_dbl(sX, reinterpret_cast<const T*>(st + L::OFF_EX), sY, reinterpret_cast<const T*>(st + L::OFF_EY),
                                 sWt, reinterpret_cast<const T*>(st + L::OFF_EW), u0, zacc);
            } else {
                sfor<0, PS>([&](auto q_) {
                    constexpr int Q = q_;
                    if (part == Q) {
                        sfor<0, NCH>([&](auto c_) {
                            constexpr int C = c_;
                            forward_item<Q, C>(sX, sY, sWt, u0 + C * MULG, zacc);
                        });
                    }
                });
            }
            if constexpr (MODE != MODE_BATCH) {
                if (hi >= 0) {                       // the chunk ends: close its last node and its empty tail
                    flush(node);
                    prev = -1;
                    if constexpr (MODE == MODE_DET) zero_nodes(node + 1, hi);
                }
            }
        }
        const long long node = h[1];             // (batch mode: the row)
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
                group_sync(bar_id, G);
            }
            if constexpr (PRODUCER) release_stage<MODE, false>(sm, g, stage, lane);
        } else {
            // every thread is done with this stage: it may be refilled
            if constexpr (PRODUCER) release_stage<MODE, false>(sm, g, stage, lane);
            else group_sync(bar_id, G);
        }
    }
    if constexpr (MODE == MODE_BATCH) {
        if (tg == 0) bulk_wait_all<0>();
    }
}

// ---------------------------------------------------------------- backward

// Channel u's inputs, read once per edge (phase 0) and kept in registers across the phases.
template <int Q, int C, class XR, class YR>
__device__ __forceinline__ void backward_load_inputs(const T* __restrict__ sX, const T* __restrict__ sY, int u,
                                                     XR& xr, YR& yr) {
    sfor<0, N_IN1>([&](auto a_) {
        constexpr int a = a_;
        if constexpr (bwd_part_uses_in1(Q, a)) {
            const bool live = (IN1_MUL[a] == CHANNELS) || (u < IN1_MUL[a]);
#pragma unroll
            for (int i = 0; i < IN1_D[a]; ++i)
                xr[C * XPC + XR_OFF[a] + i] = live ? sX[IN1_OFF[a] + u * IN1_D[a] + i] : (T)0;
        }
    });
    if constexpr (Y_IN_REGS) {
        sfor<0, N_IN2>([&](auto b_) {
            constexpr int b = b_;
            if constexpr (bwd_part_uses_in2(Q, b)) {
#pragma unroll
                for (int j = 0; j < IN2_D[b]; ++j) yr[IN2_OFF[b] + j] = sY[IN2_OFF[b] + j];
            }
        });
    }
}

// Instructions of partition Q that are staged in phase PH.  sWt / sdZ point at the stage's weight and
// output-gradient parts, which start at weight W_PH_BEGIN[PH] / column Z_PH_BEGIN[PH] of the full rows.
template <int Q, int C, int PH, class XR, class YR, class DXA, class DYA>
__device__ __forceinline__ void backward_item(const XR& xr, const YR& yr, const T* __restrict__ sY,
                                              const T* __restrict__ sWt, const T* __restrict__ sdZ, int u,
                                              long long item, const UvuParams& p, T* __restrict__ dw_acc,
                                              T* __restrict__ dy_slot, int lane, DXA& dxacc, DYA& dyreg) {
    constexpr int WBASE = W_PH_BEGIN[PH], ZBASE = Z_PH_BEGIN[PH];
    T* dwrow = SHARED_W ? dw_acc : p.dW + item * (long long)W_NUMEL;
    sfor<0, N_INSTR>([&](auto p_) {
        constexpr int P = p_;
        if constexpr (BWD_PART_OF_INSTR[P] == Q && BWD_PHASE_OF_INSTR[P] == PH) {
            constexpr int a = I_IN1[P], b = I_IN2[P], o = I_OUT[P];
            constexpr int D1 = IN1_D[a], D2 = IN2_D[b], D3 = OUT_D[o], M2 = IN2_MUL[b];
            const bool live = (IN1_MUL[a] == CHANNELS) || (u < IN1_MUL[a]);
            T gz[D3];
#pragma unroll
            for (int k = 0; k < D3; ++k) gz[k] = live ? sdZ[OUT_OFF[o] - ZBASE + u * D3 + k] : (T)0;
            const T* x = &xr[C * XPC + XR_OFF[a]];
            if constexpr (M2 == 1) {
                T av[D1], bv[D2];
#pragma unroll
                for (int i = 0; i < D1; ++i) av[i] = (T)0;
#pragma unroll
                for (int j = 0; j < D2; ++j) bv[j] = (T)0;
                const T w = live ? (UNIT_W ? (T)1 : sWt[weight_offset<P>(u, 0) - WBASE]) : (T)0;
                if constexpr (Y_IN_REGS) {
                    cg_backward<P>(x, &yr[IN2_OFF[b]], gz, av, bv);
                } else {
                    T y[D2];
#pragma unroll
                    for (int j = 0; j < D2; ++j) y[j] = sY[IN2_OFF[b] + j];
                    cg_backward<P>(x, y, gz, av, bv);
                }
                T tw = (T)0;
#pragma unroll
                for (int i = 0; i < D1; ++i) {
                    tw = fma(x[i], av[i], tw);
                    dxacc[C * XPC + XR_OFF[a] + i] = fma(w, av[i], dxacc[C * XPC + XR_OFF[a] + i]);
                }
                if (live) {
                    if constexpr (SHARED_W) dwrow[weight_offset<P>(u, 0)] += tw;
                    else if constexpr (!UNIT_W) __stcs(dwrow + weight_offset<P>(u, 0), tw);   // written once, never re-read here
                }
                if constexpr (Y_IN_REGS) {
#pragma unroll
                    for (int j = 0; j < D2; ++j) dyreg[IN2_OFF[b] + j] = fma(w, bv[j], dyreg[IN2_OFF[b] + j]);
                } else {
#pragma unroll
                    for (int j = 0; j < D2; ++j) {
                        const T s = warp_sum(w * bv[j]);
                        if (lane == 0) dy_slot[IN2_OFF[b] + j] += s;
                    }
                }
            } else {
#pragma unroll 1
                for (int v = 0; v < M2; ++v) {
                    T y[D2], bv[D2], av[D1];
#pragma unroll
                    for (int j = 0; j < D2; ++j) { y[j] = sY[IN2_OFF[b] + v * D2 + j]; bv[j] = (T)0; }
#pragma unroll
                    for (int i = 0; i < D1; ++i) av[i] = (T)0;
                    const T w = live ? (UNIT_W ? (T)1 : sWt[weight_offset<P>(u, v) - WBASE]) : (T)0;
                    cg_backward<P>(x, y, gz, av, bv);
                    T tw = (T)0;
#pragma unroll
                    for (int i = 0; i < D1; ++i) {
                        tw = fma(x[i], av[i], tw);
                        dxacc[C * XPC + XR_OFF[a] + i] = fma(w, av[i], dxacc[C * XPC + XR_OFF[a] + i]);
                    }
                    if (live) {
                        if constexpr (SHARED_W) dwrow[weight_offset<P>(u, v)] += tw;
                        else if constexpr (!UNIT_W) __stcs(dwrow + weight_offset<P>(u, v), tw);
                    }
                    // reduce this (instruction, v) over the warp's channels; lane 0 owns the warp's slot
#pragma unroll
                    for (int j = 0; j < D2; ++j) {
                        const T s = warp_sum(w * bv[j]);
                        if (lane == 0) dy_slot[IN2_OFF[b] + v * D2 + j] += s;
                    }
                }
            }
        }
    });
}

constexpr int DYREG = Y_IN_REGS ? Y_DIM : 1;

template <int MODE>
__device__ void run_backward(const UvuParams& p, const Smem<true, MODE>& sm, int g, int tg) {
    using L = StageLayout<true>;
    using SM = Smem<true, MODE>;
    const int S = sm.stages;
    const int part = tg / MULG;
    const int u0 = tg % MULG;
    const int lane = tg & 31;
    const int warp = tg >> 5;
    const bool issuer = tg < 32;
    const long long total_groups = (long long)gridDim.x * NG;
    const long long gid = (long long)blockIdx.x * NG + g;
    const int bar_id = 1 + g;

    const T* sWshared = reinterpret_cast<const T*>(sm.shared_w());
    unsigned char* ex = sm.extra(g);
    T* dxbuf = reinterpret_cast<T*>(ex);                           // [PS][XB/ELEM]
    T* dyslots = reinterpret_cast<T*>(ex + SM::DXBUF);             // [DY_RING][WARPS_PER_GROUP][YB/ELEM]
    T* dwacc = reinterpret_cast<T*>(ex + SM::DXBUF + SM::DYSLOT);  // [W_NUMEL] (shared weights)
    constexpr int XS = XB / ELEM, YS = YB / ELEM;

    if constexpr (SHARED_W) {
        for (int i = tg; i < W_NUMEL; i += G) dwacc[i] = (T)0;
    }

    T dxacc[XPC * NCH];
#pragma unroll
    for (int i = 0; i < XPC * NCH; ++i) dxacc[i] = (T)0;
    T xr[XPC * NCH];
    T yr[Y_IN_REGS ? Y_DIM : 1];
    T dyreg[DYREG];

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

    // without a producer warp the group's first warp stages items S - 1 ahead; an edge is NPH items
    ItemWalker<MODE, true> walker(p, total_groups, gid, lane);
    long long issued = 0;
    bool more = true;
    int next_phase = 0;
    long long ce = 0, cs = 0, cr = 0, clo = -1, chi = -1;
    auto issue_next = [&]() {
        if (!more) return;
        if (next_phase == 0) {
            more = walker.next(ce, cs, cr, clo, chi);
            if (!more) {
                if (lane == 0) *reinterpret_cast<volatile long long*>(sm.total(g)) = issued;
                return;
            }
        }
        issue_item<MODE, true>(p, sm, g, (int)(issued % S), lane, ce, cs, cr, clo, chi, next_phase);
        ++issued;
        next_phase = (next_phase + 1) % NPH;
    };
    if constexpr (!PRODUCER) {
        if (issuer) {
            for (int i = 0; i < S - 1; ++i) issue_next();
        }
    }
    group_sync(bar_id, G);   // also publishes the cleared shared-weight accumulator
    int* arrivals = sm.arrivals(g);

    long long prev = -1;
    long long next_unwritten = 0;
    // optional cycle accounting, compiled in only when the descriptor says so (flags bit 4: p.ws is a counter
    // buffer): first thread of CTA 0's first group
    const bool prof = UVU_PROFILE && (p.flags & 16) && blockIdx.x == 0 && g == 0 && tg == 0;
    unsigned long long prof_wait = 0, prof_items = 0;
    const long long prof_begin = prof ? clock64() : 0;
    for (long long it = 0;; ++it) {
        const int stage = (int)(it % S);
        const int ph = (int)(it % NPH);
        const long long edge_it = it / NPH;
        if constexpr (!PRODUCER) {
            if (issuer) issue_next();
        }
        const long long prof_t0 = prof ? clock64() : 0;
        const int got = acquire_item<MODE, true>(p, sm, g, it);
        if (prof) {
            prof_wait += (unsigned long long)(clock64() - prof_t0);
            ++prof_items;
        }
        if (got != 0) break;
        const long long* h = sm.hdr(g, stage);
        const unsigned char* st = sm.stage(g, stage);
        const long long item = h[0];
        const long long node = h[1];  // sender
        const long long lo = h[2], hi = h[3];
        const T* sX = reinterpret_cast<const T*>(st + L::OFF_X);
        const T* sY = reinterpret_cast<const T*>(st + L::OFF_Y);
        const T* sWt = SHARED_W ? sWshared : reinterpret_cast<const T*>(st + L::OFF_W);
        const T* sdZ = reinterpret_cast<const T*>(st + L::OFF_DZ);
        const int ring = (int)(edge_it % DY_RING);
        T* slot = dyslots + (ring * WARPS_PER_GROUP + warp) * YS;
        const bool last_phase = ph == NPH - 1;

        if (ph == 0) {
            if constexpr (MODE != MODE_BATCH) {
                if (lo >= 0) next_unwritten = lo;
                if (prev >= 0 && node != prev) {
                    flush(prev);
                    if constexpr (MODE == MODE_DET) next_unwritten = prev + 1 > next_unwritten ? prev + 1 : next_unwritten;
                }
                if constexpr (MODE == MODE_DET) {
                    if (next_unwritten < node) zero_nodes(next_unwritten, node);
                    next_unwritten = node + 1;
                }
                prev = node;
            }
            if constexpr (!Y_IN_REGS) {
                for (int j = lane; j < Y_DIM; j += 32) slot[j] = (T)0;
                __syncwarp();
            }
#pragma unroll
            for (int j = 0; j < DYREG; ++j) dyreg[j] = (T)0;
            sfor<0, PS>([&](auto q_) {
                constexpr int Q = q_;
                if (part == Q) {
                    sfor<0, NCH>([&](auto c_) {
                        constexpr int C = c_;
                        backward_load_inputs<Q, C>(sX, sY, u0 + C * MULG, xr, yr);
                    });
                }
            });
        }
        sfor<0, NPH>([&](auto ph_) {
            constexpr int PH = ph_;
            if (ph == PH) {
                sfor<0, PS>([&](auto q_) {
                    constexpr int Q = q_;
                    if (part == Q) {
                        sfor<0, NCH>([&](auto c_) {
                            constexpr int C = c_;
                            backward_item<Q, C, PH>(xr, yr, sY, sWt, sdZ, u0 + C * MULG, item, p, dwacc, slot, lane,
                                                    dxacc, dyreg);
                        });
                    }
                });
            }
        });
        if (!last_phase) {
            // more of this edge follows in the next stage; hand this one back
            if constexpr (PRODUCER) release_stage<MODE, true>(sm, g, stage, lane);
            else group_sync(bar_id, G);
            continue;
        }
        if constexpr (Y_IN_REGS) {
            constexpr int SHIFT = 5 - log2_int(next_pow2(Y_DIM));
            warp_reduce_vector<Y_DIM>(dyreg, lane);
            const int j = lane >> SHIFT;
            if ((lane & ((1 << SHIFT) - 1)) == 0 && j < Y_DIM) slot[j] = dyreg[0];
        }
        const T* slots = dyslots + ring * WARPS_PER_GROUP * YS;
        auto sum_dy = [&](int first, int step) {   // fixed order over the warps' partials
            for (int j = first; j < Y_DIM; j += step) {
                T s = (T)0;
#pragma unroll
                for (int w = 0; w < WARPS_PER_GROUP; ++w) s += slots[w * YS + j];
                p.dY[item * (long long)Y_DIM + j] = s;
            }
        };
        if constexpr (MODE == MODE_BATCH) {
            if constexpr (PRODUCER) release_stage<MODE, true>(sm, g, stage, lane);
            flush(item);  // two group barriers, which also order the dY partials (and release the stage)
            sum_dy(tg, G);
        } else if constexpr (!PRODUCER) {
            group_sync(bar_id, G);
            if (hi >= 0) {
                flush(node);
                prev = -1;
                if constexpr (MODE == MODE_DET) zero_nodes(node + 1, hi);
            }
            sum_dy(tg, G);
        } else {
            // no per-item barrier: the warp that arrives last sums the partials of the item
            __syncwarp();
            int last = 0;
            if (lane == 0) {
                mbar_arrive(sm.empty(g, stage));
                __threadfence_block();
                last = atomicAdd(arrivals + ring, 1) == WARPS_PER_GROUP - 1;
            }
            last = __shfl_sync(0xffffffffu, last, 0);
            if (last) {
                __threadfence_block();
                sum_dy(lane, 32);
                __syncwarp();
                if (lane == 0) arrivals[ring] = 0;
            }
            if (hi >= 0) {
                flush(node);
                prev = -1;
                if constexpr (MODE == MODE_DET) zero_nodes(node + 1, hi);
            }
        }
    }
    if constexpr (SHARED_W) {
        // every (u, v, instruction) slot was accumulated by exactly one thread of the group
        group_sync(bar_id, G);
        T* out = p.ws + gid * (long long)W_NUMEL;
        for (int i = tg; i < W_NUMEL; i += G) out[i] = dwacc[i];
    } else if (prof) {
        unsigned long long* out = reinterpret_cast<unsigned long long*>(p.ws);
        out[0] = (unsigned long long)(clock64() - prof_begin);   // consumer: total cycles
        out[1] = prof_wait;                                      // ... of which waiting for staged rows
        out[2] = prof_items;                                     // staged items (edges x phases)
    }
}

// ---------------------------------------------------------------- backward, receiver order (convolution)
//
// The sender-order backward pass above stages the receiver's output-gradient row (Z_DIM values) once per
// edge; for channel-wise products that row is several times larger than everything else an edge needs, and
// moving it from L2 into shared memory per edge is what bounds that kernel.  This pass walks the edges in
// the order of the forward pass instead (runs of equal receivers): a thread keeps its channel's slice of
// dZ[receiver] in registers for the whole run, an edge stages only X[sender], Y and W, and dW and dY leave
// per edge as before.  The gradient of the first input cannot be accumulated here (one sender's edges are
// spread over many runs), so every edge emits its dX row:
//   deterministic: to scratch row `edge` (p.ws), summed afterwards per sender in sender_perm order by
//                  oeq_sum_sender_rows -- a fixed order, bit-reproducible;
//   atomic:        added into dX[sender] by one bulk reduction (element-wise add performed at L2).
// One thread per channel, all instructions (PS == 1, NCH == 1), second input in registers.

constexpr int ZPC_ALL = []() { int n = 0; for (int o = 0; o < N_OUT; ++o) n += OUT_D[o]; return n > 0 ? n : 1; }();
constexpr int out_reg_off(int o) { int n = 0; for (int q = 0; q < o; ++q) n += OUT_D[q]; return n; }
// Output irreps whose first value has index >= GZ_REGS (descriptor) keep their dZ slice in shared memory
// instead of registers: a run's slice may not fit the register budget of a CTA with staging warps.
constexpr int GZ_FIRST_SMEM = []() {
    for (int o = 0; o < N_OUT; ++o)
        if (out_reg_off(o) >= GZ_REGS) return out_reg_off(o);
    return ZPC_ALL;
}();
constexpr int GZ_IN_REGS = GZ_FIRST_SMEM;

template <int MODE>
__device__ void run_backward_recv(const UvuParams& p, const Smem<true, MODE, true>& sm, int g, int tg) {
    using SM = Smem<true, MODE, true>;
    using L = typename SM::L;
    static_assert(PS == 1 && NCH == 1 && Y_IN_REGS && !SHARED_W, "receiver-order backward: one thread per channel");
    static_assert(!DBLC || !UNIT_W, "second derivatives need the weight array");
    const int S = sm.stages;
    const int u = tg;
    const int lane = tg & 31;
    const int warp = tg >> 5;
    const bool issuer = tg < 32;
    const long long total_groups = (long long)gridDim.x * NG;
    const long long gid = (long long)blockIdx.x * NG + g;
    const int bar_id = 1 + g;
    constexpr int XS = XB / ELEM, YS = YB / ELEM;

    unsigned char* ex = sm.extra(g);
    T* dxrows = reinterpret_cast<T*>(ex);                          // [2][XS]
    T* dyslots = reinterpret_cast<T*>(ex + SM::DXBUF);             // [DY_RING][WARPS_PER_GROUP][YS]
    const bool dx_bulk = p.flags & 32;                             // atomic mode: dX rows meet the 16-byte rule

    T gz[GZ_IN_REGS > 0 ? GZ_IN_REGS : 1];
    T yr[Y_DIM], dyreg[Y_DIM];
    T* gzs = reinterpret_cast<T*>(ex + SM::DXBUF + SM::DYSLOT);    // [ZPC_ALL - GZ_IN_REGS][G]

    ItemWalker<MODE, false> walker(p, total_groups, gid, lane);
    long long issued = 0;
    bool more = true;
    auto issue_next = [&]() {
        if (!more) return;
        if constexpr (EPI > 1) {
            static_assert(EPI == 1 || (!PRODUCER && !DBLC), "runs of edges: self-staging walks");
            long long e0, s_i, r_i, lo, hi;
            int cnt;
            more = walker.next_block(e0, cnt, s_i, r_i, lo, hi);
            if (more) {
                issue_block<MODE>(p, sm, g, (int)(issued % S), lane, e0, cnt, s_i, r_i, lo, hi);
                ++issued;
            } else if (lane == 0) {
                *reinterpret_cast<volatile long long*>(sm.total(g)) = issued;
            }
        } else {
            long long e, s, r, lo, hi;
            more = walker.next(e, s, r, lo, hi);
            if (more) {
                // header slot 2 carries the sender (the forward pass keeps a node bound there)
                issue_item<MODE, false>(p, sm, g, (int)(issued % S), lane, e, s, r, s, hi);
                ++issued;
            } else if (lane == 0) {
                *reinterpret_cast<volatile long long*>(sm.total(g)) = issued;
            }
        }
    };
    if constexpr (!PRODUCER) {
        if (issuer) {
            for (int i = 0; i < S - 1; ++i) issue_next();
        }
        group_sync(bar_id, G);
    }

    long long prev = -1;
    long long ec = 0;                    // edges processed (equals `it` unless EPI > 1)
    for (long long it = 0;; ++it) {
        const int stage = (int)(it % S);
        if constexpr (!PRODUCER) {
            if (issuer) issue_next();
        }
        if (acquire_item<MODE, false>(p, sm, g, it) != 0) break;
        const long long* h = sm.hdr(g, stage);
        const unsigned char* st = sm.stage(g, stage);
        const int n_edges = EPI > 1 ? (int)h[1] : 1;
        for (int ei = 0; ei < n_edges; ++ei, ++ec) {       // the edges of the item (one unless EPI > 1)
            const long long item = EPI > 1 ? h[0] + ei : h[0];
            const long long node = EPI > 1 ? h[4 + ei] : h[1];     // receiver
            const long long sender = EPI > 1 ? h[4 + EPI + ei] : h[2];
            const T* sX = reinterpret_cast<const T*>(st + L::OFF_X + (EPI > 1 ? ei * XB : 0));
            const T* sY = reinterpret_cast<const T*>(st + L::OFF_Y) + (EPI > 1 ? ei * Y_DIM : 0);
            const T* sWt = reinterpret_cast<const T*>(st + L::OFF_W) + (EPI > 1 ? ei * W_NUMEL : 0);
            // second derivatives: the cotangents of dX (at the sender), dY and dW of this edge
            const T* sEX = reinterpret_cast<const T*>(st + L::OFF_EX);
            const T* sEY = reinterpret_cast<const T*>(st + L::OFF_EY);
            const T* sEW = reinterpret_cast<const T*>(st + L::OFF_EW);

            if (node != prev) {
                // a new run: this channel's slice of the receiver's output gradient, kept for the whole run
                const T* zrow = p.dZ + node * (long long)Z_DIM;
                sfor<0, N_OUT>([&](auto o_) {
                    constexpr int o = o_;
                    const bool live = (OUT_MUL[o] == CHANNELS) || (u < OUT_MUL[o]);
    #pragma unroll
                    for (int k = 0; k < OUT_D[o]; ++k) {
                        const T v = live ? __ldg(zrow + OUT_OFF[o] + u * OUT_D[o] + k) : (T)0;
                        if constexpr (out_reg_off(o) < GZ_REGS) gz[out_reg_off(o) + k] = v;
                        else gzs[(out_reg_off(o) - GZ_FIRST_SMEM + k) * G + u] = v;    // private to this thread
                    }
                });
                prev = node;
            }
    #pragma unroll
            for (int j = 0; j < Y_DIM; ++j) {
                yr[j] = sY[j];
                dyreg[j] = (T)0;
            }
            T* dwrow = p.dW + item * (long long)W_NUMEL;
            T* dxrow = dxrows + (ec & 1) * XS;
            const bool row_to_smem = MODE == MODE_DET || dx_bulk;
            // instructions grouped by their first-input irrep: only that block of X and of dX is live at a time,
            // and the block of the dX row leaves the registers as soon as its last instruction is done
            sfor<0, N_IN1>([&](auto a_) {
                constexpr int a = a_;
                constexpr int D1 = IN1_D[a];
                const bool live = (IN1_MUL[a] == CHANNELS) || (u < IN1_MUL[a]);
                T x[D1], dxa[D1];
                T ex[DBLC ? D1 : 1];
    #pragma unroll
                for (int i = 0; i < D1; ++i) {
                    x[i] = live ? sX[IN1_OFF[a] + u * D1 + i] : (T)0;
                    dxa[i] = (T)0;
                    if constexpr (DBLC) ex[i] = live ? sEX[IN1_OFF[a] + u * D1 + i] : (T)0;
                }
                sfor<0, N_INSTR>([&](auto p_) {
                    constexpr int P = p_;
                    if constexpr (I_IN1[P] == a && DBLC) {
                        // gx = w A(ey) + ew A(y),  gy = B(w ex + ew x),  gw = <ex, A(y)> + <x, A(ey)>  with
                        // A_i(v) = sum_j v_j P_ij, B_j(v) = sum_i v_i P_ij, P_ij = sum_k C_ijk dZ_k
                        constexpr int b = I_IN2[P], o = I_OUT[P];
                        constexpr int D2 = IN2_D[b];
                        const T w = live ? sWt[weight_offset<P>(u, 0)] : (T)0;
                        const T ew = live ? sEW[weight_offset<P>(u, 0)] : (T)0;
                        T r[D1], ay[D1], aey[D1], bv[D2], eyv[D2];
    #pragma unroll
                        for (int i = 0; i < D1; ++i) {
                            r[i] = fma(w, ex[i], ew * x[i]);
                            ay[i] = (T)0;
                            aey[i] = (T)0;
                        }
    #pragma unroll
                        for (int j = 0; j < D2; ++j) {
                            bv[j] = (T)0;
                            eyv[j] = sEY[IN2_OFF[b] + j];      // one address for the whole warp: a broadcast read
                        }
                        if constexpr (out_reg_off(o) < GZ_REGS) {
                            cg_backward_dbl<P>(r, &yr[IN2_OFF[b]], eyv, &gz[out_reg_off(o)], ay, aey, bv);
                        } else {
                            T gs[OUT_D[o]];
    #pragma unroll
                            for (int k = 0; k < OUT_D[o]; ++k) gs[k] = gzs[(out_reg_off(o) - GZ_FIRST_SMEM + k) * G + u];
                            cg_backward_dbl<P>(r, &yr[IN2_OFF[b]], eyv, gs, ay, aey, bv);
                        }
                        T tw = (T)0;
    #pragma unroll
                        for (int i = 0; i < D1; ++i) {
                            tw = fma(ex[i], ay[i], tw);
                            tw = fma(x[i], aey[i], tw);
                            dxa[i] = fma(w, aey[i], dxa[i]);
                            dxa[i] = fma(ew, ay[i], dxa[i]);
                        }
                        if (live) __stcs(dwrow + weight_offset<P>(u, 0), tw);
    #pragma unroll
                        for (int j = 0; j < D2; ++j) dyreg[IN2_OFF[b] + j] += bv[j];
                    } else if constexpr (I_IN1[P] == a) {
                        constexpr int b = I_IN2[P], o = I_OUT[P];
                        constexpr int D2 = IN2_D[b];
                        T av[D1], bv[D2];
    #pragma unroll
                        for (int i = 0; i < D1; ++i) av[i] = (T)0;
    #pragma unroll
                        for (int j = 0; j < D2; ++j) bv[j] = (T)0;
                        const T w = live ? (UNIT_W ? (T)1 : sWt[weight_offset<P>(u, 0)]) : (T)0;
                        if constexpr (out_reg_off(o) < GZ_REGS) {
                            cg_backward<P>(x, &yr[IN2_OFF[b]], &gz[out_reg_off(o)], av, bv);
                        } else {
                            // this output irrep's slice of dZ is parked in shared memory ([value][channel]: no conflicts)
                            T gs[OUT_D[o]];
    #pragma unroll
                            for (int k = 0; k < OUT_D[o]; ++k) gs[k] = gzs[(out_reg_off(o) - GZ_FIRST_SMEM + k) * G + u];
                            cg_backward<P>(x, &yr[IN2_OFF[b]], gs, av, bv);
                        }
                        T tw = (T)0;
    #pragma unroll
                        for (int i = 0; i < D1; ++i) {
                            tw = fma(x[i], av[i], tw);
                            dxa[i] = fma(w, av[i], dxa[i]);
                        }
                        if constexpr (!UNIT_W) {
                            if (live) __stcs(dwrow + weight_offset<P>(u, 0), tw);
                        }
    #pragma unroll
                        for (int j = 0; j < D2; ++j) dyreg[IN2_OFF[b] + j] = fma(w, bv[j], dyreg[IN2_OFF[b] + j]);
                    }
                });
                if (live) {
    #pragma unroll
                    for (int i = 0; i < D1; ++i) {
                        if (row_to_smem) dxrow[IN1_OFF[a] + u * D1 + i] = dxa[i];
                        else if constexpr (any_part_uses_in1(a))
                            red_add(p.dX + sender * (long long)X_DIM + IN1_OFF[a] + u * D1 + i, dxa[i]);
                    }
                }
            });
            // the stage has been read: hand it back
            if constexpr (PRODUCER) release_stage<MODE, false>(sm, g, stage, lane);
            const int ring = (int)(ec % DY_RING);
            {
                constexpr int SHIFT = 5 - log2_int(next_pow2(Y_DIM));
                warp_reduce_vector<Y_DIM>(dyreg, lane);
                const int j = lane >> SHIFT;
                if ((lane & ((1 << SHIFT) - 1)) == 0 && j < Y_DIM) dyslots[(ring * WARPS_PER_GROUP + warp) * YS + j] = dyreg[0];
            }
            // the bulk copy that read the other dX row buffer (issued one edge ago) leaves this one alone; the copy
            // that read *this* buffer two edges ago was waited for before the previous barrier
            if (row_to_smem) {
                fence_async_smem();                     // this thread's part of the row, visible to the bulk copy
                if (tg == 0) bulk_wait_read<0>();       // every earlier row copy has read its buffer: the next edge may overwrite it
            }
            group_sync(bar_id, G);
            if (tg == 0 && row_to_smem) {
                if constexpr (MODE == MODE_DET) {
                    bulk_s2g(reinterpret_cast<unsigned char*>(p.ws) + item * (long long)XB, dxrow, XB);
                } else {
                    if constexpr (ELEM == 4) bulk_red_add_f32(reinterpret_cast<float*>(p.dX) + sender * (long long)X_DIM, dxrow, XB);
                    else bulk_red_add_f64(reinterpret_cast<double*>(p.dX) + sender * (long long)X_DIM, dxrow, XB);
                }
                bulk_commit();
            }
            {
                const T* slots = dyslots + ring * WARPS_PER_GROUP * YS;
                const int first = G >= 64 ? tg - 32 : tg;      // the second warp sums when there is one
                if (first >= 0 && first < Y_DIM) {
                    T sum = (T)0;
    #pragma unroll
                    for (int w = 0; w < WARPS_PER_GROUP; ++w) sum += slots[w * YS + first];
                    p.dY[item * (long long)Y_DIM + first] = sum;
                }
            }
        }
    }
    if (tg == 0) bulk_wait_all<0>();
}

// dX[s] = (or +=) the sum of the scratch rows of the edges that s sends, in sender_perm order, for the edges
// of [e_lo, e_hi) whose rows `temp` holds (pitch XB bytes).  Work is dealt to `warps` warps in chunks of
// the sender-ordered edge list; chunk ends are moved forward to the next sender boundary, so a sender's
// edges are never split between two warps: every row of dX has one writer and a fixed summation order.
// 32 positions are examined at a time; positions whose edge lies outside the range cost one coalesced
// load and a ballot.  `first`: store the rows of the senders met (the host has cleared dX, so nodes that
// send nothing stay zero); otherwise add.
__device__ __forceinline__ long long align_sender(const long long* cols, const long long* perm, long long n, long long t,
                                                  int lane) {
    if (t <= 0) return 0;
    if (t >= n) return n;
    for (long long base = t; base < n + 32; base += 32) {
        const long long idx = base + lane;
        bool boundary = idx >= n;
        if (!boundary) boundary = cols[perm[idx]] != cols[perm[idx - 1]];
        const unsigned ballot = __ballot_sync(0xffffffffu, boundary);
        if (ballot) return base + (__ffs(ballot) - 1);
    }
    return n;
}

__device__ void sum_sender_rows(const T* __restrict__ temp, T* __restrict__ dX, const long long* __restrict__ cols,
                                const long long* __restrict__ perm, long long n_items, long long e_lo, long long e_hi,
                                bool first, int chunk, long long warps, long long wid, int lane) {
    constexpr int VEC = 16 / ELEM;                                  // elements per 16-byte load
    constexpr int XS = XB / ELEM;
    constexpr int NV = (XS / VEC + 31) / 32;                        // 16-byte pieces per lane
    T acc[NV * VEC];
#pragma unroll
    for (int i = 0; i < NV * VEC; ++i) acc[i] = (T)0;
    auto flush = [&](long long node) {
        T* xrow = dX + node * (long long)X_DIM;
#pragma unroll
        for (int v = 0; v < NV; ++v) {
            const int base = (lane + 32 * v) * VEC;
            if (base < X_DIM) {
#pragma unroll
                for (int q = 0; q < VEC; ++q)
                    if (base + q < X_DIM) {
                        if (first) xrow[base + q] = acc[v * VEC + q];
                        else xrow[base + q] += acc[v * VEC + q];
                    }
            }
        }
#pragma unroll
        for (int i = 0; i < NV * VEC; ++i) acc[i] = (T)0;
    };
    const long long n_chunks = (n_items + chunk - 1) / chunk;
    for (long long c = wid; c < n_chunks; c += warps) {
        const long long pos = align_sender(cols, perm, n_items, c * chunk, lane);
        const long long end = c + 1 >= n_chunks ? n_items : align_sender(cols, perm, n_items, (c + 1) * chunk, lane);
        long long prev = -1;
        for (long long base = pos; base < end; base += 32) {
            const long long k = base + lane;
            long long e = -1, s = -1;
            if (k < end) e = perm[k];
            const bool in_block = e >= e_lo && e < e_hi;
            unsigned mask = __ballot_sync(0xffffffffu, in_block);
            if (mask == 0) continue;
            if (in_block) s = cols[e];
            // Short rows: the loads of up to U rows go out together (a row at a time would pay the DRAM latency
            // per row); the rows are still added one after the other, in order.
            constexpr int U = (NV * VEC <= 16) ? 4 : (NV * VEC <= 32 ? 2 : 1);
            while (mask) {
                long long ej[U], sj[U];
                T val[U][NV * VEC];
                int n = 0;
#pragma unroll
                for (int q = 0; q < U; ++q) {
                    ej[q] = 0; sj[q] = -1;
                    if (mask) {
                        const int src = __ffs(mask) - 1;
                        mask &= mask - 1;
                        ej[q] = __shfl_sync(0xffffffffu, e, src);
                        sj[q] = __shfl_sync(0xffffffffu, s, src);
                        n = q + 1;
                    }
                }
#pragma unroll
                for (int q = 0; q < U; ++q) {
                    if (q < n) {
                        const T* row = temp + (ej[q] - e_lo) * (long long)XS;
#pragma unroll
                        for (int v = 0; v < NV; ++v) {
                            const int b4 = (lane + 32 * v) * VEC;
                            if (b4 < XS) {
                                if constexpr (ELEM == 4) {
                                    const float4 t = __ldcs(reinterpret_cast<const float4*>(row + b4));
                                    val[q][v * VEC + 0] = t.x; val[q][v * VEC + 1] = t.y; val[q][v * VEC + 2] = t.z; val[q][v * VEC + 3] = t.w;
                                } else {
                                    const double2 t = __ldcs(reinterpret_cast<const double2*>(row + b4));
                                    val[q][v * VEC + 0] = t.x; val[q][v * VEC + 1] = t.y;
                                }
                            } else {
#pragma unroll
                                for (int c = 0; c < VEC; ++c) val[q][v * VEC + c] = (T)0;
                            }
                        }
                    }
                }
#pragma unroll
                for (int q = 0; q < U; ++q) {
                    if (q < n) {
                        if (prev >= 0 && sj[q] != prev) flush(prev);
                        prev = sj[q];
#pragma unroll
                        for (int i = 0; i < NV * VEC; ++i) acc[i] += val[q][i];
                    }
                }
            }
        }
        if (prev >= 0) flush(prev);
    }
}

template <int MODE>
__device__ __forceinline__ void uvu_body_recv(const UvuParams& p) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    Smem<true, MODE, true> sm(smem_raw, p.stages);
    const int tid = threadIdx.x;
    if (tid == 0) {
        const bool any_elem = EPI > 1 || !(p.flags & 1) || !(p.flags & 2) || (!(p.flags & 4) && !UNIT_W);
        for (int g = 0; g < NG; ++g) {
            for (int s = 0; s < p.stages; ++s) {
                mbar_init(sm.full(g, s), 1 + (any_elem ? 32 : 0));
                mbar_init(sm.empty(g, s), WARPS_PER_GROUP);
            }
            *sm.total(g) = -1;
        }
        fence_mbar_init();
    }
    __syncthreads();
    if (tid >= NCONSUMERS + NSTAGING) {
        if constexpr (HELPER_WARPS > 0) {
            if (p.sum_items > 0)
                sum_sender_rows(p.sum_ws, p.dX, p.sum_cols, p.sum_perm, p.sum_items, p.sum_e_lo, p.sum_e_hi, p.sum_first != 0,
                                p.sum_chunk, (long long)gridDim.x * HELPER_WARPS,
                                (long long)blockIdx.x * HELPER_WARPS + ((tid - NCONSUMERS - NSTAGING) >> 5), tid & 31);
        }
        return;
    }
    if (PRODUCER && tid >= NCONSUMERS) {
        run_producer<MODE, false, true>(p, sm, (tid - NCONSUMERS) >> 5, tid & 31);
        return;
    }
    run_backward_recv<MODE>(p, sm, tid / G, tid % G);
}

// ---------------------------------------------------------------- second derivatives, batch product, one pass
//
// With Z = T(x, y, w) trilinear and the first derivatives dX, dY, dW taken against dZ, the gradient of
// <ex, dX> + <ey, dY> + <ew, dW> with respect to (x, y, w, dZ) is
//   gx = dX(ey, w) + dX(y, ew),  gy = dY(ex, w) + dY(x, ew),  gw = dW(ex, y) + dW(x, ey),
//   gdz = T(ex, y, w) + T(x, ey, w) + T(x, y, ew)
// which the reference (and this library's general path) evaluates with four backward and three forward launches
// (reference: openequivariance/implementations/TensorProductBase.py:284-296).  All seven terms share the row's
// x, y, w, dZ and the products P_ij = sum_k C_ijk dZ_k, so this kernel loads a row's seven arrays once and emits
// the four results: per instruction and (i, j) pair
//   q_j = w ey_j + ew y_j,  r_i = w ex_i + ew x_i
//   gx_i += q_j P_ij,  gy_j += r_i P_ij,  gw += (ex_i y_j + x_i ey_j) P_ij,
//   gdz_k += C_ijk (r_i y_j + w x_i ey_j)
// 7 FMAs per pair and 2 per coefficient, against 4 x (3 per pair + 1 per coefficient) + 3 x (1 + 1) composed.
// One thread per channel, per-row weights, second input of multiplicity 1 kept in registers.

struct DblLayout {
    static constexpr int OFF_X = 0;
    static constexpr int OFF_EX = OFF_X + XB;
    static constexpr int OFF_Y = OFF_EX + XB;
    static constexpr int OFF_EY = OFF_Y + YB;
    static constexpr int OFF_W = OFF_EY + YB;
    static constexpr int OFF_EW = OFF_W + WB;
    static constexpr int OFF_DZ = OFF_EW + WB;
    static constexpr int BYTES = OFF_DZ + ZB;
};

struct DblSmem {
    using L = DblLayout;
    static constexpr int DYSLOT = DY_RING * WARPS_PER_GROUP * YB;
    static constexpr int EXTRA = DYSLOT;
    static constexpr int CTRL = 128;
    unsigned char* base;
    int stages;
    __device__ DblSmem(unsigned char* b, int s) : base(b), stages(s) {}
    __device__ unsigned long long* full(int g, int s) const { return reinterpret_cast<unsigned long long*>(base) + (g * stages + s) * 2; }
    __device__ unsigned long long* empty(int g, int s) const { return full(g, s) + 1; }
    __device__ long long* hdr(int g, int s) const { return reinterpret_cast<long long*>(base + NG * stages * 16) + (g * stages + s) * 4; }
    __device__ long long* total(int g) const { return reinterpret_cast<long long*>(base + NG * stages * 48 + g * CTRL); }
    __device__ unsigned char* group_base(int g) const { return base + NG * stages * 48 + NG * CTRL + (long long)g * (stages * L::BYTES + EXTRA); }
    __device__ unsigned char* stage(int g, int s) const { return group_base(g) + s * L::BYTES; }
    __device__ unsigned char* extra(int g) const { return group_base(g) + stages * L::BYTES; }
};

// Staging warp of group g: rows gid, gid + groups, ... ; seven copies per row on the stage's barrier.
template <int INSTANCE>     // templates: compiled only in the translation unit that asks for this kernel
__device__ void run_producer_dbl(const UvuParams& p, const DblSmem& sm, int g, int lane) {
    using L = DblLayout;
    const int S = sm.stages;
    const long long groups = (long long)gridDim.x * NG, gid = (long long)blockIdx.x * NG + g;
    volatile long long* total = sm.total(g);
    long long it = 0;
    bool ok = true;
    // per array: a bulk copy when it meets the 16-byte rule (flags bit 0 X and EX, 1 Y and EY, 2 W and EW, 3 dZ),
    // element copies by the whole warp otherwise
    const int bit[7] = {1, 1, 2, 2, 4, 4, 8};
    const bool any_elem = (p.flags & 15) != 15;
    for (long long row = gid; row < p.n_items && ok; row += groups, ++it) {
        const int stage = (int)(it % S);
        if (it >= S) ok = mbar_wait(sm.empty(g, stage), (unsigned)(((it / S) - 1) & 1), p.status, ERR_WAIT_EMPTY);
        if (!ok) break;
        unsigned char* st = sm.stage(g, stage);
        unsigned long long* full = sm.full(g, stage);
        const T* src[7] = {p.X + row * X_DIM, p.EX + row * X_DIM, p.Y + row * Y_DIM, p.EY + row * Y_DIM,
                           p.W + row * (long long)W_NUMEL, p.EW + row * (long long)W_NUMEL, p.dZ + row * (long long)Z_DIM};
        const int off[7] = {L::OFF_X, L::OFF_EX, L::OFF_Y, L::OFF_EY, L::OFF_W, L::OFF_EW, L::OFF_DZ};
        const int len[7] = {X_DIM, X_DIM, Y_DIM, Y_DIM, W_NUMEL, W_NUMEL, Z_DIM};
        if (lane == 0) {
            sm.hdr(g, stage)[0] = row;
            unsigned bytes = 0;
#pragma unroll
            for (int a = 0; a < 7; ++a)
                if (p.flags & bit[a]) bytes += (unsigned)pad16(len[a] * ELEM);
            mbar_arrive_expect_tx(full, bytes);
#pragma unroll
            for (int a = 0; a < 7; ++a)
                if (p.flags & bit[a]) bulk_g2s(st + off[a], src[a], (unsigned)pad16(len[a] * ELEM), full);
        }
        if (any_elem) {
#pragma unroll
            for (int a = 0; a < 7; ++a)
                if (!(p.flags & bit[a]))
                    for (int i = lane; i < len[a]; i += 32) cp_async_elem<ELEM>((T*)(st + off[a]) + i, src[a] + i);
            cp_async_arrive_noinc(full);
        }
    }
    if (lane == 0) *total = it;
    asm volatile("cp.async.wait_all;" ::: "memory");
}

template <int INSTANCE>
__device__ void run_double_backward(const UvuParams& p, const DblSmem& sm, int g, int tg) {
    using L = DblLayout;
    static_assert(PS == 1 && NCH == 1 && Y_IN_REGS && !SHARED_W && !UNIT_W && PRODUCER, "one thread per channel");
    const int S = sm.stages;
    const int u = tg, lane = tg & 31, warp = tg >> 5;
    const int bar_id = 1 + g;
    constexpr int YS = YB / ELEM;
    T* dyslots = reinterpret_cast<T*>(sm.extra(g));
    for (long long it = 0;; ++it) {
        const int stage = (int)(it % S);
        int got = 2;
        {
            volatile long long* total = sm.total(g);
            for (unsigned spin = 0; spin < WAIT_LIMIT; ++spin) {
                if (mbar_try_wait(sm.full(g, stage), (unsigned)((it / S) & 1))) { got = 0; break; }
                const long long n = *total;
                if (n >= 0 && it >= n) { got = 1; break; }
            }
            if (got == 2 && p.status) atomicCAS(p.status, 0, ERR_WAIT_FULL);
        }
        if (got != 0) break;
        const long long row = sm.hdr(g, stage)[0];
        const unsigned char* st = sm.stage(g, stage);
        const T* sX = reinterpret_cast<const T*>(st + L::OFF_X);
        const T* sEX = reinterpret_cast<const T*>(st + L::OFF_EX);
        const T* sY = reinterpret_cast<const T*>(st + L::OFF_Y);
        const T* sEY = reinterpret_cast<const T*>(st + L::OFF_EY);
        const T* sW = reinterpret_cast<const T*>(st + L::OFF_W);
        const T* sEW = reinterpret_cast<const T*>(st + L::OFF_EW);
        const T* sdZ = reinterpret_cast<const T*>(st + L::OFF_DZ);
        T yr[Y_DIM], eyr[Y_DIM], gyreg[Y_DIM];
#pragma unroll
        for (int j = 0; j < Y_DIM; ++j) { yr[j] = sY[j]; eyr[j] = sEY[j]; gyreg[j] = (T)0; }
        T gdz[ZPC_ALL];
#pragma unroll
        for (int k = 0; k < ZPC_ALL; ++k) gdz[k] = (T)0;
        T* gwrow = p.dW + row * (long long)W_NUMEL;
        T* gxrow = p.dX + row * (long long)X_DIM;
        sfor<0, N_IN1>([&](auto a_) {
            constexpr int a = a_;
            constexpr int D1 = IN1_D[a];
            const bool live = (IN1_MUL[a] == CHANNELS) || (u < IN1_MUL[a]);
            T x[D1], ex[D1], gxa[D1];
#pragma unroll
            for (int i = 0; i < D1; ++i) {
                x[i] = live ? sX[IN1_OFF[a] + u * D1 + i] : (T)0;
                ex[i] = live ? sEX[IN1_OFF[a] + u * D1 + i] : (T)0;
                gxa[i] = (T)0;
            }
            sfor<0, N_INSTR>([&](auto p_) {
                constexpr int P = p_;
                if constexpr (I_IN1[P] == a) {
                    constexpr int b = I_IN2[P], o = I_OUT[P];
                    constexpr int D2 = IN2_D[b], D3 = OUT_D[o];
                    const T w = live ? sW[weight_offset<P>(u, 0)] : (T)0;
                    const T ew = live ? sEW[weight_offset<P>(u, 0)] : (T)0;
                    T gz[D3], q[D2], r[D1], wx[D1];
#pragma unroll
                    for (int k = 0; k < D3; ++k) gz[k] = live ? sdZ[OUT_OFF[o] + u * D3 + k] : (T)0;
#pragma unroll
                    for (int j = 0; j < D2; ++j) q[j] = fma(w, eyr[IN2_OFF[b] + j], ew * yr[IN2_OFF[b] + j]);
#pragma unroll
                    for (int i = 0; i < D1; ++i) { r[i] = fma(w, ex[i], ew * x[i]); wx[i] = w * x[i]; }
                    T gw = (T)0, pij = (T)0, tij = (T)0;
                    sfor<CG_BEGIN[P], CG_BEGIN[P + 1]>([&](auto n) {
                        constexpr int N = n;
                        constexpr int I = CG_I[N], J = CG_J[N], K = CG_K[N];
                        if constexpr (cg_pair_first<P, N>()) {
                            pij = (T)CG_V[N] * gz[K];
                            tij = fma(r[I], yr[IN2_OFF[b] + J], wx[I] * eyr[IN2_OFF[b] + J]);
                        } else {
                            pij = fma((T)CG_V[N], gz[K], pij);
                        }
                        gdz[out_reg_off(o) + K] = fma((T)CG_V[N], tij, gdz[out_reg_off(o) + K]);
                        if constexpr (cg_pair_last<P, N>()) {
                            gxa[I] = fma(q[J], pij, gxa[I]);
                            gyreg[IN2_OFF[b] + J] = fma(r[I], pij, gyreg[IN2_OFF[b] + J]);
                            gw = fma(fma(ex[I], yr[IN2_OFF[b] + J], x[I] * eyr[IN2_OFF[b] + J]), pij, gw);
                        }
                    });
                    if (live) __stcs(gwrow + weight_offset<P>(u, 0), gw);
                }
            });
            if (live) {
#pragma unroll
                for (int i = 0; i < D1; ++i) __stcs(gxrow + IN1_OFF[a] + u * D1 + i, gxa[i]);
            }
        });
        // the stage has been read: hand it back
        __syncwarp();
        if (lane == 0) mbar_arrive(sm.empty(g, stage));
        // gradient with respect to dZ: this channel's slice of the row
        {
            T* zrow = p.Z + row * (long long)Z_DIM;
            sfor<0, N_OUT>([&](auto o_) {
                constexpr int o = o_;
                if ((OUT_MUL[o] == CHANNELS) || (u < OUT_MUL[o])) {
#pragma unroll
                    for (int k = 0; k < OUT_D[o]; ++k) __stcs(zrow + OUT_OFF[o] + u * OUT_D[o] + k, gdz[out_reg_off(o) + k]);
                }
            });
        }
        // gradient with respect to y: over the channels of the warp, then over the warps
        const int ring = (int)(it % DY_RING);
        {
            constexpr int SHIFT = 5 - log2_int(next_pow2(Y_DIM));
            warp_reduce_vector<Y_DIM>(gyreg, lane);
            const int j = lane >> SHIFT;
            if ((lane & ((1 << SHIFT) - 1)) == 0 && j < Y_DIM) dyslots[(ring * WARPS_PER_GROUP + warp) * YS + j] = gyreg[0];
        }
        group_sync(bar_id, G);
        {
            const T* slots = dyslots + ring * WARPS_PER_GROUP * YS;
            if (tg < Y_DIM) {
                T sum = (T)0;
#pragma unroll
                for (int w2 = 0; w2 < WARPS_PER_GROUP; ++w2) sum += slots[w2 * YS + tg];
                p.dY[row * (long long)Y_DIM + tg] = sum;
            }
        }
    }
}

template <int INSTANCE>
__device__ __forceinline__ void uvu_body_dbl(const UvuParams& p) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    DblSmem sm(smem_raw, p.stages);
    const int tid = threadIdx.x;
    if (tid == 0) {
        const bool any_elem = (p.flags & 15) != 15;
        for (int g = 0; g < NG; ++g) {
            for (int s = 0; s < p.stages; ++s) {
                mbar_init(sm.full(g, s), 1 + (any_elem ? 32 : 0));
                mbar_init(sm.empty(g, s), WARPS_PER_GROUP);
            }
            *sm.total(g) = -1;
        }
        fence_mbar_init();
    }
    __syncthreads();
    if (tid >= NCONSUMERS) {
        run_producer_dbl<INSTANCE>(p, sm, (tid - NCONSUMERS) >> 5, tid & 31);
        return;
    }
    run_double_backward<INSTANCE>(p, sm, tid / G, tid % G);
}

// ---------------------------------------------------------------- kernel body

template <int MODE, bool BWD>
__device__ __forceinline__ void uvu_body(const UvuParams& p) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    Smem<BWD, MODE> sm(smem_raw, p.stages);
    const int tid = threadIdx.x;

    if (tid == 0) {
        const bool any_elem = (EPI > 1 && !BWD) || !(p.flags & 1) || !(p.flags & 2) || (!(p.flags & 4) && !SHARED_W && !UNIT_W) ||
                              (BWD && !(p.flags & 8));
        for (int g = 0; g < NG; ++g) {
            for (int s = 0; s < p.stages; ++s) {
                mbar_init(sm.full(g, s), 1 + (any_elem ? 32 : 0));
                mbar_init(sm.empty(g, s), WARPS_PER_GROUP);
            }
            *sm.total(g) = -1;
            for (int r = 0; r < DY_RING; ++r) sm.arrivals(g)[r] = 0;
        }
        fence_mbar_init();
    }
    if constexpr (SHARED_W) {
        T* sw = reinterpret_cast<T*>(sm.shared_w());
        for (int i = tid; i < W_NUMEL; i += NTHREADS) sw[i] = p.W[i];
    }
    __syncthreads();

    if (PRODUCER && tid >= NCONSUMERS) {
        run_producer<MODE, BWD>(p, sm, (tid - NCONSUMERS) >> 5, tid & 31);
        return;
    }
    const int g = tid / G, tg = tid % G;
    if constexpr (BWD) run_backward<MODE>(p, sm, g, tg);
    else run_forward<MODE>(p, sm, g, tg);
}

}  // namespace oeq

// One entry point per translation unit, selected by OEQ_KERNEL (other kernel files include this
// header for its building blocks and define OEQ_UVU_NO_ENTRY).
#ifndef OEQ_UVU_NO_ENTRY

extern "C" __global__ void __launch_bounds__(oeq::NTHREADS, oeqd::MIN_CTAS) oeq_uvu_kernel(const oeq::UvuParams p) {
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
#elif OEQ_KERNEL == OEQ_K_BWD_RECV_DET
    oeq::uvu_body_recv<oeq::MODE_DET>(p);
#elif OEQ_KERNEL == OEQ_K_BWD_RECV_ATOMIC
    oeq::uvu_body_recv<oeq::MODE_ATOMIC>(p);
#elif OEQ_KERNEL == OEQ_K_DBL_BATCH
    oeq::uvu_body_dbl<0>(p);
#elif OEQ_KERNEL == OEQ_K_DBLC_Z_DET
    oeq::uvu_body<oeq::MODE_DET, false>(p);
#elif OEQ_KERNEL == OEQ_K_DBLC_Z_ATOMIC
    oeq::uvu_body<oeq::MODE_ATOMIC, false>(p);
#elif OEQ_KERNEL == OEQ_K_DBLC_G_DET
    oeq::uvu_body_recv<oeq::MODE_DET>(p);
#elif OEQ_KERNEL == OEQ_K_DBLC_G_ATOMIC
    oeq::uvu_body_recv<oeq::MODE_ATOMIC>(p);
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

#if OEQ_KERNEL == OEQ_K_BWD_RECV_DET || OEQ_KERNEL == OEQ_K_DBLC_G_DET || OEQ_KERNEL == OEQ_K_DBLC_G_ATOMIC
// Clears `bytes` bytes (a multiple of 4) at a 4-byte aligned address.  A kernel rather than a memset call: a
// memset may be served by a copy engine, where it would queue behind host transfers that other streams have
// in flight and stall the stream that runs the backward pass.
extern "C" __global__ void oeq_clear(unsigned int* ptr, unsigned long long words) {
    const unsigned long long stride = (unsigned long long)gridDim.x * blockDim.x;
    unsigned long long i = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x;
    // 16-byte stores over the aligned middle, words at the ragged ends
    const unsigned long long head = ((16 - (reinterpret_cast<unsigned long long>(ptr) & 15)) & 15) / 4;
    const unsigned long long h = head < words ? head : words;
    const unsigned long long quads = (words - h) / 4;
    uint4* mid = reinterpret_cast<uint4*>(ptr + h);
    for (unsigned long long q = i; q < quads; q += stride) mid[q] = make_uint4(0u, 0u, 0u, 0u);
    if (i < h) ptr[i] = 0u;
    const unsigned long long tail0 = h + quads * 4;
    if (i < words - tail0) ptr[tail0 + i] = 0u;
}

// The row sum of the deterministic receiver-order backward pass as a launch of its own (the last block of
// edges, or every block when the launches carry no helper warps): see sum_sender_rows.
extern "C" __global__ void __launch_bounds__(256) oeq_sum_sender_rows(const oeq::UvuParams p) {
    oeq::sum_sender_rows(reinterpret_cast<const oeqd::T*>(p.ws), p.dX, p.cols, p.perm, p.n_items, p.e_lo, p.e_hi,
                         (p.flags & 64) != 0, p.chunk, (long long)gridDim.x * (blockDim.x >> 5),
                         (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), threadIdx.x & 31);
}
#endif
#endif  // OEQ_UVU_NO_ENTRY
