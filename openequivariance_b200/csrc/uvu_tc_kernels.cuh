// Forward pass of the fused "uvu" graph convolution on the 5th-generation tensor cores (tcgen05, TMEM
// accumulators), FP32 in / FP32 out with 3xTF32 error compensation, for problems whose widest
// multiplicity is 65..128 and whose second input has multiplicity 1.
//
// For one edge the channel-wise product is, per channel u,
//     t[u, (p,k)] = sum_i x[u,i] * M[i, (p,k)],      M[i, (p,k)] = sum_j c^p_ijk y_j,
//     Z[node, o(p), u, k] += w[p,u] * t[u, (p,k)]
// i.e. a [128 x K] x [K x N] product with the channels as rows, K = the per-channel width of the first
// input (16 for l <= 3) and N = the per-channel width of all paths' outputs.  M depends on the edge
// only, not on the channel, so it is formed once per edge (its entries are the Clebsch-Gordan
// nonzeros contracted with Y) instead of once per channel.
//
// One CTA per SM, three roles:
//   * the staging warp walks the CTA's edges (same chunked deal as the FMA kernels) and stages X (gathered
//     at the sender), W and Y rows with bulk async copies;
//   * eight consumer warps, thread = (output partition, channel): split the channel's X values into
//     hi/lo and store them as the swizzled K-major A tile of the edge, and write their one or two
//     entries of M (coefficients in registers), split the same way, into the swizzled B tile; one edge
//     later they read their
//     columns of the edge's accumulator from tensor memory, scale by the weights and add into the
//     receiver's row held in registers (written once per receiver, as in the FMA kernel: same order of
//     summation, bit-reproducible);
//   * one thread issues tcgen05.mma (M = 128, N = padded column count, K = 8) three times per K step
//     (hi.hi + hi.lo + lo.hi) and commits to an mbarrier.
// A and B tiles and the accumulator are double buffered, so conversion, MMA and epilogue of
// neighbouring edges overlap.  Every wait is bounded; on expiry the role records a code in *status and
// stops, and the CTA still frees its tensor memory.
//
// Replaces the forward kernels of the reference's convolution templates
// (openequivariance/templates/loop_unroll_conv_det.cuh:64-141, loop_unroll_conv_atomic.cuh:40-90).
#pragma once
#define OEQ_UVU_NO_ENTRY
#include "uvu_kernels.cuh"
#include "tc_common.cuh"

namespace oeq {

constexpr int UTC_PARTS = PS;                  // consumer partitions (each owns some output irreps)
constexpr int UTC_CONSUMERS = 128 * UTC_PARTS;
constexpr int UTC_CONSUMER_WARPS = UTC_CONSUMERS / 32;
constexpr int UTC_WARP_STAGE = UTC_CONSUMER_WARPS, UTC_WARP_MMA = UTC_CONSUMER_WARPS + 1;
constexpr int UTC_THREADS = UTC_CONSUMERS + 2 * 32;
constexpr int ERR_UTC_A = 21, ERR_UTC_DFREE = 23, ERR_UTC_D = 24;

// ---- columns of the product: path p owns columns [TC_COL_BEGIN[p], TC_COL_BEGIN[p] + 2 l_out + 1); the paths
// of consumer partition q are contiguous and start at TC_PART_COL[q], a multiple of 16 (tables from the host)
constexpr int UTC_NPAD = TC_PART_COL[UTC_PARTS];
constexpr int UTC_DCOLS = UTC_NPAD <= 32 ? 32 : UTC_NPAD <= 64 ? 64 : UTC_NPAD <= 128 ? 128 : 256;   // per accumulator
constexpr int UTC_TMEM_COLS = 2 * UTC_DCOLS;
constexpr int UTC_KSTEPS = (XPC + 7) / 8;
constexpr int utc_path_of_col(int c) {          // -1: padding column
    for (int p = 0; p < N_INSTR; ++p)
        if (c >= TC_COL_BEGIN[p] && c < TC_COL_BEGIN[p] + OUT_D[I_OUT[p]]) return p;
    return -1;
}
constexpr int utc_paths_of_part(int q) {
    int n = 0;
    for (int p = 0; p < N_INSTR; ++p) n += FWD_PART_OF_OUT[I_OUT[p]] == q;
    return n;
}
constexpr int utc_path_rank(int p) {            // index of path p among the paths of its partition
    int n = 0;
    for (int r = 0; r < p; ++r) n += FWD_PART_OF_OUT[I_OUT[r]] == FWD_PART_OF_OUT[I_OUT[p]];
    return n;
}

// ---- shared memory map (1024-byte aligned base): [A x2][B x2][control][stages]
constexpr int UTC_A_HALF = 128 * 128;                 // [128 rows x 32 tf32] swizzled tile
constexpr int UTC_A_BYTES = 2 * UTC_A_HALF;           // hi + lo
constexpr int UTC_B_HALF = UTC_NPAD * 128;
constexpr int UTC_B_BYTES = 2 * UTC_B_HALF;
constexpr int UTC_OFF_A = 0;
constexpr int UTC_OFF_B = UTC_OFF_A + 2 * UTC_A_BYTES;
constexpr int UTC_OFF_CTRL = UTC_OFF_B + 2 * UTC_B_BYTES;
constexpr int UTC_CTRL_BYTES = 512;
constexpr int UTC_OFF_STAGE = UTC_OFF_CTRL + UTC_CTRL_BYTES;
constexpr int UTC_STAGE_BYTES = XB + WB + YB;           // X, W, Y rows of one edge
constexpr int UTC_MAX_STAGES = 4;

struct UtcCtrl {
    unsigned long long* full;      // [UTC_MAX_STAGES]  X and W rows of the stage have landed
    unsigned long long* empty;     // [UTC_MAX_STAGES]  consumers are done with the stage
    unsigned long long* a_ready;   // [2] A and B tiles written by the consumers
    unsigned long long* d_ready;   // [2] accumulator complete (and A, B tiles read)
    unsigned long long* d_free;    // [2] accumulator read by the consumers
    long long* hdr;                // [UTC_MAX_STAGES][4] edge, receiver, chunk node range markers
    volatile long long* total;     // number of edges of this CTA, -1 until known
    unsigned* tmem_slot;
    __device__ explicit UtcCtrl(unsigned char* smem) {
        unsigned long long* b = reinterpret_cast<unsigned long long*>(smem + UTC_OFF_CTRL);
        full = b; empty = b + UTC_MAX_STAGES;
        a_ready = b + 2 * UTC_MAX_STAGES; d_ready = a_ready + 2; d_free = d_ready + 2;
        hdr = reinterpret_cast<long long*>(d_free + 2);
        total = hdr + 4 * UTC_MAX_STAGES;
        tmem_slot = reinterpret_cast<unsigned*>(const_cast<long long*>(total) + 1);
    }
};
static_assert((2 * UTC_MAX_STAGES + 8) * 8 + 4 * UTC_MAX_STAGES * 8 + 16 <= UTC_CTRL_BYTES, "control block too small");

// Optional cycle accounting per role (CTA 0 only), written to p.ws when the host passes a buffer there.
// Sums are kept in registers and stored once when the role ends.
struct UtcProf {
    unsigned long long* out;
    long long t0;
    unsigned long long acc[8];
    __device__ UtcProf(const UvuParams& p, int base, bool leader)
        : out((p.ws && blockIdx.x == 0 && leader) ? reinterpret_cast<unsigned long long*>(p.ws) + base : nullptr), t0(0) {
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = 0;
    }
    __device__ __forceinline__ void start() { if (out) t0 = clock64(); }
    __device__ __forceinline__ void stop(int slot) { if (out) acc[slot] += (unsigned long long)(clock64() - t0); }
    __device__ __forceinline__ void add(int slot, unsigned long long v) { if (out) acc[slot] += v; }
    __device__ __forceinline__ void flush() {
        if (out) {
#pragma unroll
            for (int i = 0; i < 8; ++i) out[i] += acc[i];
        }
    }
};

// Wait for `bar` or for the end of the CTA's edge sequence.  0: completed, 1: no such edge, 2: gave up.
__device__ __forceinline__ int utc_wait_or_end(unsigned long long* bar, unsigned parity, const UtcCtrl& c, long long item,
                                               int* status, int code) {
    for (unsigned spin = 0; spin < WAIT_LIMIT; ++spin) {
        if (mbar_try_wait(bar, parity)) return 0;
        const long long n = *c.total;
        if (n >= 0 && item >= n) return 1;
    }
    if (status) atomicCAS(status, 0, code);
    return 2;
}

// ---------------------------------------------------------------------------- staging warp
template <int MODE>
__device__ void utc_stager(const UvuParams& p, unsigned char* smem, const UtcCtrl& c, int lane) {
    const int S = p.stages;
    ItemWalker<MODE, false> walker(p, (long long)gridDim.x, (long long)blockIdx.x, lane);
    const bool xb = p.flags & 1, yb = p.flags & 2, wb = p.flags & 4;
    bool ok = true;
    long long it = 0;
    UtcProf prof(p, 32, lane == 0);
    const long long t_begin = clock64();
    while (ok) {
        long long e, s, r, lo, hi;
        prof.start();
        const bool got = walker.next(e, s, r, lo, hi);
        prof.stop(2);
        if (!got) break;
        const int stage = (int)(it % S);
        prof.start();
        if (it >= S) ok = mbar_wait(c.empty + stage, (unsigned)(((it / S) - 1) & 1), p.status, ERR_WAIT_EMPTY);
        prof.stop(1);
        if (!ok) break;
        unsigned char* st = smem + UTC_OFF_STAGE + stage * UTC_STAGE_BYTES;
        const T* xsrc = p.X + s * (long long)X_DIM;
        const T* wsrc = p.W + e * (long long)W_NUMEL;
        const T* ysrc = p.Y + e * (long long)Y_DIM;
        if (lane == 0) {
            long long* h = c.hdr + 4 * stage;
            h[0] = e; h[1] = r; h[2] = lo; h[3] = hi;
            mbar_arrive_expect_tx(c.full + stage, (xb ? XB : 0) + (wb ? WB : 0) + (yb ? YB : 0));
            const unsigned long long keep = l2_policy_evict_last(), stream = l2_policy_evict_first();
            if (wb) bulk_g2s_hint(st + XB, wsrc, WB, c.full + stage, stream);
            if (xb) bulk_g2s_hint(st, xsrc, XB, c.full + stage, keep);
            if (yb) bulk_g2s_hint(st + XB + WB, ysrc, YB, c.full + stage, stream);
        }
        if (!xb || !wb || !yb) {
            if (!xb) for (int i = lane; i < X_DIM; i += 32) cp_async_elem<ELEM>((T*)st + i, xsrc + i);
            if (!wb) for (int i = lane; i < W_NUMEL; i += 32) cp_async_elem<ELEM>((T*)(st + XB) + i, wsrc + i);
            if (!yb) for (int i = lane; i < Y_DIM; i += 32) cp_async_elem<ELEM>((T*)(st + XB + WB) + i, ysrc + i);
            cp_async_arrive_noinc(c.full + stage);
        }
        ++it;
    }
    prof.add(0, (unsigned long long)(clock64() - t_begin));
    prof.add(3, (unsigned long long)it);
    prof.flush();
    if (lane == 0) *c.total = it;
    asm volatile("cp.async.wait_all;" ::: "memory");
}

// ---------------------------------------------------------------------------- MMA issuer (one thread)
__device__ void utc_mma(const UvuParams& p, unsigned char* smem, const UtcCtrl& c, unsigned tmem_base) {
    constexpr unsigned IDESC = tc_instr_desc(UTC_NPAD);
    const unsigned long long a_desc0 = tc_smem_desc(smem_u32(smem + UTC_OFF_A));
    const unsigned long long b_desc0 = tc_smem_desc(smem_u32(smem + UTC_OFF_B));
    UtcProf prof(p, 16, true);
    const long long t_begin = clock64();
    for (long long n = 0;; ++n) {
        const int b = (int)(n & 1);
        const long long use = n >> 1;
        prof.start();
        const int rc = utc_wait_or_end(c.a_ready + b, (unsigned)(use & 1), c, n, p.status, ERR_UTC_A);
        prof.stop(1);
        if (rc != 0) break;
        prof.start();
        const bool df = !(use > 0 && !mbar_wait(c.d_free + b, (unsigned)((use - 1) & 1), p.status, ERR_UTC_DFREE));
        prof.stop(3);
        if (!df) break;
        prof.start();
        tc_fence_after();
        // descriptors differ from the base ones only in the start-address field (16-byte units)
        const unsigned long long da_hi = a_desc0 + (unsigned long long)((b * UTC_A_BYTES) >> 4), da_lo = da_hi + (UTC_A_HALF >> 4);
        const unsigned long long db_hi = b_desc0 + (unsigned long long)((b * UTC_B_BYTES) >> 4), db_lo = db_hi + (UTC_B_HALF >> 4);
        const unsigned tmem_d = tmem_base + (unsigned)(b * UTC_DCOLS);
#pragma unroll
        for (int kk = 0; kk < UTC_KSTEPS; ++kk) {
            tc_mma(tmem_d, da_hi + 2 * kk, db_hi + 2 * kk, IDESC, kk == 0 ? 0u : 1u);
            tc_mma(tmem_d, da_hi + 2 * kk, db_lo + 2 * kk, IDESC, 1);
            tc_mma(tmem_d, da_lo + 2 * kk, db_hi + 2 * kk, IDESC, 1);
        }
        tc_commit(c.d_ready + b);
        prof.stop(4);
    }
    prof.add(0, (unsigned long long)(clock64() - t_begin));
    prof.flush();
}

// ---------------------------------------------------------------------------- consumer warps
// Partition Q: the consumers that own the output irreps with FWD_PART_OF_OUT == Q.
template <int MODE, int Q>
__device__ void utc_consumer(const UvuParams& p, unsigned char* smem, const UtcCtrl& c, unsigned tmem_base, int u) {
    const int S = p.stages;
    const int lane = u & 31, quarter = (u >> 5) & 3;
    constexpr int COL0 = TC_PART_COL[Q];
    constexpr int NCHUNK = (TC_PART_COL[Q + 1] - COL0) / 16;
    constexpr int NPATHS = utc_paths_of_part(Q);
    // chunks (4 columns) of the A tile that this partition converts
    constexpr int CH_TOTAL = 2 * UTC_KSTEPS;
    constexpr int CH_LO = Q * CH_TOTAL / UTC_PARTS, CH_HI = (Q + 1) * CH_TOTAL / UTC_PARTS;
    T zacc[ZPC_MAX];
#pragma unroll
    for (int i = 0; i < ZPC_MAX; ++i) zacc[i] = (T)0;
    // this thread's entries of the per-edge matrix M (B tile): offsets, term indices and coefficients
    constexpr int NE = (TCM_N + UTC_CONSUMERS - 1) / UTC_CONSUMERS;
    const int gtid = Q * 128 + u;
    int m_off[NE], m_j[NE][TCM_TMAX];
    float m_c[NE][TCM_TMAX];
#pragma unroll
    for (int q = 0; q < NE; ++q) {
        const int e = q * UTC_CONSUMERS + gtid;
        const int ec = e < TCM_N ? e : TCM_N - 1;
        m_off[q] = e < TCM_N ? TCM_OFF_DEV[ec] : -1;
#pragma unroll
        for (int t = 0; t < TCM_TMAX; ++t) {
            m_j[q][t] = TCM_J_DEV[ec * TCM_TMAX + t];
            m_c[q][t] = TCM_C_DEV[ec * TCM_TMAX + t];
        }
    }

    auto flush = [&](long long node) {
        T* zrow = p.Z + node * (long long)Z_DIM;
        for_each_out<Q, 0>(u, [&](int zoff, int reg) {
            if constexpr (MODE == MODE_DET) zrow[zoff] = zacc[reg];
            else red_add(zrow + zoff, zacc[reg]);
            zacc[reg] = (T)0;
        });
    };
    auto zero_nodes = [&](long long lo, long long hi) {       // partition 0 clears rows of nodes without edges
        if constexpr (Q == 0) {
            for (long long node = lo; node < hi; ++node) {
                T* zrow = p.Z + node * (long long)Z_DIM;
                for (int i = u; i < Z_DIM; i += 128) zrow[i] = (T)0;
            }
        }
    };

    long long prev = -1, next_unwritten = 0;
    bool more = true;
    UtcProf prof(p, 8 * Q, u == 0);
    const long long t_begin = clock64();
    // operands of edge n: this thread's entries of the B tile and its share of the A tile
    auto convert = [&](long long n) {
        prof.start();
        if (more) {
            // this thread's entries of the B tile: M = Clebsch-Gordan coefficients contracted with the edge's Y
            const T* sY = reinterpret_cast<const T*>(smem + UTC_OFF_STAGE + (int)(n % S) * UTC_STAGE_BYTES + XB + WB);
            unsigned char* bhi = smem + UTC_OFF_B + (int)(n & 1) * UTC_B_BYTES;
            unsigned char* blo = bhi + UTC_B_HALF;
#pragma unroll
            for (int q = 0; q < NE; ++q) {
                if (m_off[q] >= 0) {
                    float acc = 0.f;
#pragma unroll
                    for (int t = 0; t < TCM_TMAX; ++t) acc = fmaf(m_c[q][t], sY[m_j[q][t]], acc);
                    const float h = tf32_hi(acc);
                    *reinterpret_cast<float*>(bhi + m_off[q]) = h;
                    *reinterpret_cast<float*>(blo + m_off[q]) = acc - h;
                }
            }
        }
        if (more && CH_HI > CH_LO) {
            // this partition's share of the channel's row of the A tile, split into hi and lo
            const T* sX = reinterpret_cast<const T*>(smem + UTC_OFF_STAGE + (int)(n % S) * UTC_STAGE_BYTES);
            float x[4 * CH_TOTAL];
#pragma unroll
            for (int i = 0; i < 4 * CH_TOTAL; ++i) x[i] = 0.f;
            sfor<0, N_IN1>([&](auto a_) {
                constexpr int a = a_;
                if constexpr (any_part_uses_in1(a)) {
                    const bool live = (IN1_MUL[a] == CHANNELS) || (u < IN1_MUL[a]);
                    sfor<0, IN1_D[a]>([&](auto i_) {
                        constexpr int col = XR_OFF[a] + i_;
                        if constexpr (col >= 4 * CH_LO && col < 4 * CH_HI)
                            x[col] = live ? sX[IN1_OFF[a] + u * IN1_D[a] + i_] : 0.f;
                    });
                }
            });
            unsigned char* hi = smem + UTC_OFF_A + (int)(n & 1) * UTC_A_BYTES;
            unsigned char* lo = hi + UTC_A_HALF;
            const int row_off = (u >> 3) * 1024 + (u & 7) * 128;
#pragma unroll
            for (int q = CH_LO; q < CH_HI; ++q) {
                float4 h, l;
                // the low part is exact in FP32; the tensor core reads its leading 10 mantissa bits
                h.x = tf32_hi(x[4 * q + 0]); l.x = x[4 * q + 0] - h.x;
                h.y = tf32_hi(x[4 * q + 1]); l.y = x[4 * q + 1] - h.y;
                h.z = tf32_hi(x[4 * q + 2]); l.z = x[4 * q + 2] - h.z;
                h.w = tf32_hi(x[4 * q + 3]); l.w = x[4 * q + 3] - h.w;
                const int off = row_off + (((q ^ (u & 7)) & 7) << 4);
                *reinterpret_cast<float4*>(hi + off) = h;
                *reinterpret_cast<float4*>(lo + off) = l;
            }
        }
        if (more) {
            fence_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(c.a_ready + (int)(n & 1));
        }
        prof.stop(3);
    };
    // accumulator of edge m: scale by the weights, add into the receiver's row
    auto epilogue = [&](long long m) -> bool {
            const int b = (int)(m & 1), stage = (int)(m % S);
            // weights of this partition's paths for the channel (the stage is still held)
            const T* sWt = reinterpret_cast<const T*>(smem + UTC_OFF_STAGE + stage * UTC_STAGE_BYTES + XB);
            T w[NPATHS > 0 ? NPATHS : 1];
            sfor<0, N_INSTR>([&](auto p_) {
                constexpr int P = p_;
                if constexpr (FWD_PART_OF_OUT[I_OUT[P]] == Q) {
                    constexpr int a = I_IN1[P];
                    const bool live = (IN1_MUL[a] == CHANNELS) || (u < IN1_MUL[a]);
                    w[utc_path_rank(P)] = live ? sWt[weight_offset<P>(u, 0)] : (T)0;
                }
            });
            const long long* h = c.hdr + 4 * stage;
            const long long node = h[1], lo = h[2], hi = h[3];
            prof.start();
            const bool dr = mbar_wait(c.d_ready + b, (unsigned)((m >> 1) & 1), p.status, ERR_UTC_D);
            prof.stop(2);
            if (!dr) return false;
            prof.start();
            tc_fence_after();
            // a warp may only read the TMEM lanes of its own quarter: 32 * (warp index mod 4)
            const unsigned taddr = tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)(b * UTC_DCOLS + COL0);
            unsigned v[16 * (NCHUNK > 0 ? NCHUNK : 1)];
            const long long t_ld = clock64();
#pragma unroll
            for (int q = 0; q < NCHUNK; ++q) tc_load16(taddr + (unsigned)(16 * q), v + 16 * q);
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
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            prof.add(6, (unsigned long long)(clock64() - t_ld));
            sfor<0, 16 * NCHUNK>([&](auto j_) {
                constexpr int col = COL0 + j_;
                constexpr int P = utc_path_of_col(col);
                if constexpr (P >= 0) {
                    constexpr int k = col - TC_COL_BEGIN[P];
                    constexpr int o = I_OUT[P];
                    zacc[ZR_OFF[o] + k] = fma(w[utc_path_rank(P)], __uint_as_float(v[j_]), zacc[ZR_OFF[o] + k]);
                }
            });
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(c.d_free + b);
                mbar_arrive(c.empty + stage);
            }
            if (hi >= 0) {                       // the chunk ends: close its last node and its empty tail
                flush(node);
                prev = -1;
                if constexpr (MODE == MODE_DET) zero_nodes(node + 1, hi);
            }
            prof.stop(4);
        return true;
    };
    // partition 0 converts first and then drains the previous edge, partition 1 the other way round, so
    // that the two consumer warps of a scheduler are in different phases and hide each other's latency
    for (long long n = 0;; ++n) {
        if (more) {
            prof.start();
            const int rc = utc_wait_or_end(c.full + (int)(n % S), (unsigned)((n / S) & 1), c, n, p.status, ERR_WAIT_FULL);
            prof.stop(1);
            if (rc == 2) return;
            if (rc == 1) more = false;
        }
        if constexpr (Q == 0) {
            if (more) convert(n);
            if (n >= 1 && !epilogue(n - 1)) return;
        } else {
            if (n >= 1 && !epilogue(n - 1)) return;
            if (more) convert(n);
        }
        if (!more) break;
    }
    prof.add(0, (unsigned long long)(clock64() - t_begin));
    prof.flush();
}

// ---------------------------------------------------------------------------- kernel body
template <int MODE>
__device__ void uvu_tc_forward(const UvuParams& p) {
    static_assert(sizeof(T) == 4, "the tensor-core forward pass is FP32");
    static_assert(MULG == 128 && NCH == 1 && UTC_PARTS >= 1 && UTC_PARTS <= 2, "thread = (partition, channel)");
    extern __shared__ __align__(16) unsigned char smem_raw[];
    // the 128-byte swizzle pattern repeats every 1024 bytes: operand tiles must start on that boundary
    unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    const UtcCtrl c(smem);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    if (tid == 0) {
        const bool any_elem = !(p.flags & 1) || !(p.flags & 2) || !(p.flags & 4);
        for (int s = 0; s < UTC_MAX_STAGES; ++s) {
            mbar_init(c.full + s, 1 + (any_elem ? 32 : 0));
            mbar_init(c.empty + s, UTC_CONSUMER_WARPS);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(c.a_ready + b, UTC_CONSUMER_WARPS);
            mbar_init(c.d_ready + b, 1);
            mbar_init(c.d_free + b, UTC_CONSUMER_WARPS);
        }
        *c.total = -1;
        fence_mbar_init();
    }
    // entries of the B tiles that no Clebsch-Gordan coefficient reaches stay zero for the whole kernel
    for (int i = tid; i < 2 * UTC_B_BYTES / 16; i += UTC_THREADS)
        reinterpret_cast<float4*>(smem + UTC_OFF_B)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    fence_async_smem();
    if (warp == UTC_WARP_MMA) {   // the MMA warp owns the tensor memory allocation
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(c.tmem_slot)),
                     "n"(UTC_TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem_base = *reinterpret_cast<volatile unsigned*>(c.tmem_slot);

    if (warp < UTC_CONSUMER_WARPS) {
        sfor<0, UTC_PARTS>([&](auto q_) {
            constexpr int Q = q_;
            if (tid / 128 == Q) utc_consumer<MODE, Q>(p, smem, c, tmem_base, tid % 128);
        });
    } else if (warp == UTC_WARP_STAGE) {
        utc_stager<MODE>(p, smem, c, lane);
    } else {
        if (lane == 0) utc_mma(p, smem, c, tmem_base);
        __syncwarp();
    }
    tc_fence_before();
    __syncthreads();
    if (warp == UTC_WARP_MMA) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "n"(UTC_TMEM_COLS) : "memory");
    }
}

}  // namespace oeq

#define OEQ_K_FWD_DET_TC 30
#define OEQ_K_FWD_ATOMIC_TC 31

extern "C" __global__ void __launch_bounds__(oeq::UTC_THREADS, 1) oeq_uvu_tc_kernel(const oeq::UvuParams p) {
#if OEQ_KERNEL == OEQ_K_FWD_DET_TC
    oeq::uvu_tc_forward<oeq::MODE_DET>(p);
#elif OEQ_KERNEL == OEQ_K_FWD_ATOMIC_TC
    oeq::uvu_tc_forward<oeq::MODE_ATOMIC>(p);
#else
#error "OEQ_KERNEL must select one of the tensor-core uvu kernels"
#endif
}
