// "uvw" (fully connected) tensor product kernels, FP32 / FP64 FMA path.
//
// Replaces the uvw branches of the reference's generated kernels and its warp-level
// matmul (openequivariance/templates/loop_unroll_tp.cuh:11-18,54-83,176-219,
// openequivariance/templates/wmm.cuh:1-88).
//
//   Z[b,o,w,k] += sum_{u,v} W_p[u,v,w] * T_p[b,u,v,k],   T_p[b,u,v,k] = sum_{ij} C_p[i,j,k] x[b,u,i] y[b,v,j]
//
// A CTA works on a tile of TILE_R batch rows.  Per instruction and per chunk of UVC
// (u,v) pairs it (1) forms T for the tile in shared memory with the Clebsch-Gordan
// constants unrolled, and (2) contracts T with the weights as a register-tiled small
// GEMM, so a weight is read once per tile instead of once per row.  The backward pass
// forms dT = W . dZ the same way, derives dX and dY from dT, and accumulates the weight
// gradient of a shared weight tensor into a per-CTA slice of the caller's scratch
// buffer (summed afterwards in a fixed order: bit-reproducible), or stores it per row.
#pragma once
#include "oeq_common.cuh"

namespace oeq {
using namespace oeqd;

struct UvwParams {
    const T* X;
    const T* Y;
    const T* W;
    T* Z;
    const T* dZ;
    T* dX;
    T* dY;
    T* dW;
    T* ws;  // [gridDim.x][W_NUMEL] partial weight gradients (shared weights)
    long long batch;
    int* status;
    int skip_dw;   // shared weights: the weight gradient is computed elsewhere, leave dW and ws alone
};

constexpr int NT = UVW_THREADS;
constexpr int RT = 4;  // rows per thread in the register tiles

// Offset of W_p[u,v,w] in the kernel weight layout: 32-wide chunks ordered (u,v,w)-chunk
// major, each chunk stored [v][u][w].
template <int P>
__device__ __forceinline__ int uvw_weight_offset(int u, int v, int w) {
    constexpr int MU = IN1_MUL[I_IN1[P]], MV = IN2_MUL[I_IN2[P]], MW = OUT_MUL[I_OUT[P]];
    if constexpr (MU <= 32 && MV <= 32 && MW <= 32) {
        return W_OFF[P] + (v * MU + u) * MW + w;
    } else {
        const int uc = u >> 5, ul = u & 31, vc = v >> 5, vl = v & 31, wc = w >> 5, wl = w & 31;
        const int ulen = (MU - (uc << 5)) < 32 ? (MU - (uc << 5)) : 32;
        const int vlen = (MV - (vc << 5)) < 32 ? (MV - (vc << 5)) : 32;
        const int wlen = (MW - (wc << 5)) < 32 ? (MW - (wc << 5)) : 32;
        return W_OFF[P] + (uc << 5) * MV * MW + ulen * ((vc << 5) * MW + vlen * (wc << 5)) +
               (vl * ulen + ul) * wlen + wl;
    }
}

template <int P, class XA, class YA, class TA>
__device__ __forceinline__ void uvw_cg_forward(const XA& x, const YA& y, TA& t) {
    sfor<CG_BEGIN[P], CG_BEGIN[P + 1]>([&](auto n) {
        constexpr int N = n;
        t[CG_K[N]] = fma(x[CG_I[N]] * y[CG_J[N]], (T)CG_V[N], t[CG_K[N]]);
    });
}

// Shared memory layout (element counts come from the descriptor).
struct UvwSmem {
    T* xs;   // [TILE_R][X_DIM]
    T* ys;   // [TILE_R][Y_DIM]
    T* zs;   // [TILE_R][Z_DIM]        forward: output tile; backward: dZ tile
    T* tb;   // [UVC][TILE_R][DMAX]    T (forward) / dT (backward) chunk
    T* gx;   // [TILE_R][X_DIM]        backward: dX tile
    T* gy;   // [TILE_R][Y_DIM]        backward: dY tile
    T* zt;   // [MWMAX][TILE_R][DMAX]  backward: dZ block of the current output irrep, w-major
    T* tt;   // [UVC][TILE_R][DMAX]    backward: T chunk (tb holds dT)
};

__device__ __forceinline__ UvwSmem carve(unsigned char* raw, bool bwd) {
    UvwSmem s;
    T* p = reinterpret_cast<T*>(raw);
    auto take = [&](int n) { T* q = p; p += (n + 3) / 4 * 4; return q; };
    s.xs = take(TILE_R * X_DIM);
    s.ys = take(TILE_R * Y_DIM);
    s.zs = take(TILE_R * Z_DIM);
    s.tb = take(UVC * TILE_R * DMAX);
    s.gx = s.gy = s.zt = s.tt = nullptr;
    if (bwd) {
        s.gx = take(TILE_R * X_DIM);
        s.gy = take(TILE_R * Y_DIM);
        s.zt = take(MWMAX * TILE_R * DMAX);
        s.tt = take(UVC * TILE_R * DMAX);
    }
    return s;
}

// T chunk of instruction P for (u,v) pairs [uv0, uv0+n): dst[(uv-uv0)][r][k].
template <int P>
__device__ __forceinline__ void form_t(const UvwSmem& s, T* dst, int uv0, int n, int tid) {
    constexpr int a = I_IN1[P], b = I_IN2[P], o = I_OUT[P];
    constexpr int D1 = IN1_D[a], D2 = IN2_D[b], D3 = OUT_D[o], MV = IN2_MUL[b];
    for (int idx = tid; idx < n * TILE_R; idx += NT) {
        const int r = idx % TILE_R, l = idx / TILE_R, uv = uv0 + l;
        const int u = uv / MV, v = uv % MV;
        T x[D1], y[D2], t[D3];
#pragma unroll
        for (int i = 0; i < D1; ++i) x[i] = s.xs[r * X_DIM + IN1_OFF[a] + u * D1 + i];
#pragma unroll
        for (int j = 0; j < D2; ++j) y[j] = s.ys[r * Y_DIM + IN2_OFF[b] + v * D2 + j];
#pragma unroll
        for (int k = 0; k < D3; ++k) t[k] = (T)0;
        uvw_cg_forward<P>(x, y, t);
#pragma unroll
        for (int k = 0; k < D3; ++k) dst[(l * TILE_R + r) * D3 + k] = t[k];
    }
}

__device__ __forceinline__ void load_tile(T* dst, const T* src, long long row0, long long batch, int dim, int tid) {
    const long long rows = batch - row0 < TILE_R ? batch - row0 : TILE_R;
    const int n = (int)rows * dim;
    const T* g = src + row0 * dim;
    for (int i = tid; i < TILE_R * dim; i += NT) dst[i] = i < n ? g[i] : (T)0;
}
__device__ __forceinline__ void store_tile(T* dst, const T* src, long long row0, long long batch, int dim, int tid) {
    const long long rows = batch - row0 < TILE_R ? batch - row0 : TILE_R;
    const int n = (int)rows * dim;
    T* g = dst + row0 * dim;
    for (int i = tid; i < n; i += NT) g[i] = src[i];
}

// ------------------------------------------------------------------------- forward

__device__ void uvw_forward(const UvwParams& p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const UvwSmem s = carve(smem_raw, false);
    const int tid = threadIdx.x;
    const long long tiles = (p.batch + TILE_R - 1) / TILE_R;
    for (long long tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
        const long long row0 = tile * TILE_R;
        load_tile(s.xs, p.X, row0, p.batch, X_DIM, tid);
        load_tile(s.ys, p.Y, row0, p.batch, Y_DIM, tid);
        for (int i = tid; i < TILE_R * Z_DIM; i += NT) s.zs[i] = (T)0;
        __syncthreads();
        sfor<0, N_INSTR>([&](auto p_) {
            constexpr int P = p_;
            constexpr int a = I_IN1[P], b = I_IN2[P], o = I_OUT[P];
            constexpr int D3 = OUT_D[o], MU = IN1_MUL[a], MV = IN2_MUL[b], MW = OUT_MUL[o];
            constexpr int NUV = MU * MV;
            constexpr int ITEMS = MW * (TILE_R / RT);
            // register tiles: each thread owns RT rows x D3 components of up to NACC output channels
            constexpr int NACC = (ITEMS + NT - 1) / NT;
            T acc[NACC][RT][D3];
#pragma unroll
            for (int q = 0; q < NACC; ++q)
#pragma unroll
                for (int rr = 0; rr < RT; ++rr)
#pragma unroll
                    for (int k = 0; k < D3; ++k) acc[q][rr][k] = (T)0;
            for (int uv0 = 0; uv0 < NUV; uv0 += UVC) {
                const int n = NUV - uv0 < UVC ? NUV - uv0 : UVC;
                form_t<P>(s, s.tb, uv0, n, tid);
                __syncthreads();
#pragma unroll
                for (int q = 0; q < NACC; ++q) {
                    const int item = tid + q * NT;
                    if (item < ITEMS) {
                        const int w = item % MW, rb = item / MW;
                        for (int l = 0; l < n; ++l) {
                            const int uv = uv0 + l;
                            const int off = uvw_weight_offset<P>(uv / MV, uv % MV, w);
                            const T* tsrc = s.tb + (l * TILE_R + rb * RT) * D3;
                            if constexpr (SHARED_W) {
                                const T wv = p.W[off];
#pragma unroll
                                for (int rr = 0; rr < RT; ++rr)
#pragma unroll
                                    for (int k = 0; k < D3; ++k) acc[q][rr][k] = fma(wv, tsrc[rr * D3 + k], acc[q][rr][k]);
                            } else {
#pragma unroll
                                for (int rr = 0; rr < RT; ++rr) {
                                    const long long row = row0 + rb * RT + rr;
                                    const T wv = row < p.batch ? p.W[row * (long long)W_NUMEL + off] : (T)0;
#pragma unroll
                                    for (int k = 0; k < D3; ++k) acc[q][rr][k] = fma(wv, tsrc[rr * D3 + k], acc[q][rr][k]);
                                }
                            }
                        }
                    }
                }
                __syncthreads();
            }
#pragma unroll
            for (int q = 0; q < NACC; ++q) {
                const int item = tid + q * NT;
                if (item < ITEMS) {
                    const int w = item % MW, rb = item / MW;
#pragma unroll
                    for (int rr = 0; rr < RT; ++rr)
#pragma unroll
                        for (int k = 0; k < D3; ++k)
                            s.zs[(rb * RT + rr) * Z_DIM + OUT_OFF[o] + w * D3 + k] += acc[q][rr][k];
                }
            }
            __syncthreads();
        });
        store_tile(p.Z, s.zs, row0, p.batch, Z_DIM, tid);
        __syncthreads();
    }
}

// ------------------------------------------------------------------------- backward

__device__ void uvw_backward(const UvwParams& p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const UvwSmem s = carve(smem_raw, true);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const long long tiles = (p.batch + TILE_R - 1) / TILE_R;
    const bool with_dw = !(SHARED_W && p.skip_dw);
    T* wsl = (SHARED_W && with_dw) ? p.ws + (long long)blockIdx.x * W_NUMEL : nullptr;
    if constexpr (SHARED_W) {
        if (with_dw) {
            for (int i = tid; i < W_NUMEL; i += NT) wsl[i] = (T)0;
            __syncthreads();
        }
    }
    for (long long tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
        const long long row0 = tile * TILE_R;
        load_tile(s.xs, p.X, row0, p.batch, X_DIM, tid);
        load_tile(s.ys, p.Y, row0, p.batch, Y_DIM, tid);
        load_tile(s.zs, p.dZ, row0, p.batch, Z_DIM, tid);
        for (int i = tid; i < TILE_R * X_DIM; i += NT) s.gx[i] = (T)0;
        for (int i = tid; i < TILE_R * Y_DIM; i += NT) s.gy[i] = (T)0;
        __syncthreads();
        sfor<0, N_INSTR>([&](auto p_) {
            constexpr int P = p_;
            constexpr int a = I_IN1[P], b = I_IN2[P], o = I_OUT[P];
            constexpr int D1 = IN1_D[a], D2 = IN2_D[b], D3 = OUT_D[o];
            constexpr int MU = IN1_MUL[a], MV = IN2_MUL[b], MW = OUT_MUL[o];
            constexpr int NUV = MU * MV;
            // dZ block of this output irrep, w-major: zt[w][r][k]
            for (int idx = tid; idx < MW * TILE_R * D3; idx += NT) {
                const int k = idx % D3, r = (idx / D3) % TILE_R, w = idx / (D3 * TILE_R);
                s.zt[idx] = s.zs[r * Z_DIM + OUT_OFF[o] + w * D3 + k];
            }
            __syncthreads();
            for (int uv0 = 0; uv0 < NUV; uv0 += UVC) {
                const int n = NUV - uv0 < UVC ? NUV - uv0 : UVC;
                form_t<P>(s, s.tt, uv0, n, tid);
                // dT[l][r][k] = sum_w W[uv,w] dZ[r,w,k]: one thread per (uv, block of RT rows)
                for (int item = tid; item < n * (TILE_R / RT); item += NT) {
                    const int l = item % n, rb = item / n, uv = uv0 + l;
                    T acc[RT][D3];
#pragma unroll
                    for (int rr = 0; rr < RT; ++rr)
#pragma unroll
                        for (int k = 0; k < D3; ++k) acc[rr][k] = (T)0;
                    for (int w = 0; w < MW; ++w) {
                        const int off = uvw_weight_offset<P>(uv / MV, uv % MV, w);
                        const T* zsrc = s.zt + (w * TILE_R + rb * RT) * D3;
                        if constexpr (SHARED_W) {
                            const T wv = p.W[off];
#pragma unroll
                            for (int rr = 0; rr < RT; ++rr)
#pragma unroll
                                for (int k = 0; k < D3; ++k) acc[rr][k] = fma(wv, zsrc[rr * D3 + k], acc[rr][k]);
                        } else {
#pragma unroll
                            for (int rr = 0; rr < RT; ++rr) {
                                const long long row = row0 + rb * RT + rr;
                                const T wv = row < p.batch ? p.W[row * (long long)W_NUMEL + off] : (T)0;
#pragma unroll
                                for (int k = 0; k < D3; ++k) acc[rr][k] = fma(wv, zsrc[rr * D3 + k], acc[rr][k]);
                            }
                        }
                    }
#pragma unroll
                    for (int rr = 0; rr < RT; ++rr)
#pragma unroll
                        for (int k = 0; k < D3; ++k) s.tb[(l * TILE_R + rb * RT + rr) * D3 + k] = acc[rr][k];
                }
                __syncthreads();
                // weight gradient
                if constexpr (SHARED_W) {
                    // dW[uv,w] += sum_{r,k} T[uv,r,k] dZ[r,w,k]; the owning thread adds into the CTA's slice
                    for (int item = tid; with_dw && item < n * MW; item += NT) {
                        const int w = item % MW, l = item / MW, uv = uv0 + l;
                        const T* tsrc = s.tt + l * TILE_R * D3;
                        const T* zsrc = s.zt + w * TILE_R * D3;
                        T sum = (T)0;
#pragma unroll 4
                        for (int e = 0; e < TILE_R * D3; ++e) sum = fma(tsrc[e], zsrc[e], sum);
                        wsl[uvw_weight_offset<P>(uv / MV, uv % MV, w)] += sum;
                    }
                } else {
                    for (int item = tid; item < n * MW * TILE_R; item += NT) {
                        const int w = item % MW, l = (item / MW) % n, r = item / (MW * n), uv = uv0 + l;
                        const long long row = row0 + r;
                        if (row < p.batch) {
                            const T* tsrc = s.tt + (l * TILE_R + r) * D3;
                            const T* zsrc = s.zt + (w * TILE_R + r) * D3;
                            T sum = (T)0;
#pragma unroll
                            for (int k = 0; k < D3; ++k) sum = fma(tsrc[k], zsrc[k], sum);
                            p.dW[row * (long long)W_NUMEL + uvw_weight_offset<P>(uv / MV, uv % MV, w)] = sum;
                        }
                    }
                }
                // dX[r,u,i] += sum_{v,j,k} C y[r,v,j] dT[u,v,r,k]: one thread owns (r, u) and walks the v of
                // that u which fall inside this chunk, so the sum order is fixed.
                {
                    const int u_lo = uv0 / MV, u_n = (uv0 + n - 1) / MV - u_lo + 1;
                    for (int item = tid; item < u_n * TILE_R; item += NT) {
                        const int r = item % TILE_R, u = u_lo + item / TILE_R;
                        T dx[D1];
#pragma unroll
                        for (int i = 0; i < D1; ++i) dx[i] = (T)0;
                        for (int v = 0; v < MV; ++v) {
                            const int uv = u * MV + v;
                            if (uv < uv0 || uv >= uv0 + n) continue;
                            const int l = uv - uv0;
                            T y[D2], g[D3];
#pragma unroll
                            for (int j = 0; j < D2; ++j) y[j] = s.ys[r * Y_DIM + IN2_OFF[b] + v * D2 + j];
#pragma unroll
                            for (int k = 0; k < D3; ++k) g[k] = s.tb[(l * TILE_R + r) * D3 + k];
                            sfor<CG_BEGIN[P], CG_BEGIN[P + 1]>([&](auto n_) {
                                constexpr int N = n_;
                                dx[CG_I[N]] = fma((T)CG_V[N] * g[CG_K[N]], y[CG_J[N]], dx[CG_I[N]]);
                            });
                        }
#pragma unroll
                        for (int i = 0; i < D1; ++i) s.gx[r * X_DIM + IN1_OFF[a] + u * D1 + i] += dx[i];
                    }
                }
                // dY[r,v,j] += sum_{u,i,k} C x[r,u,i] dT[u,v,r,k]: a warp per (r, v), lanes over u, fixed-order
                // warp reduction, lane 0 accumulates.
                for (int rv = warp; rv < TILE_R * MV; rv += NT / 32) {
                    const int r = rv % TILE_R, v = rv / TILE_R;
                    T dy[D2];
#pragma unroll
                    for (int j = 0; j < D2; ++j) dy[j] = (T)0;
                    for (int u = lane; u < MU; u += 32) {
                        const int uv = u * MV + v;
                        if (uv >= uv0 && uv < uv0 + n) {
                            const int l = uv - uv0;
                            T x[D1], g[D3];
#pragma unroll
                            for (int i = 0; i < D1; ++i) x[i] = s.xs[r * X_DIM + IN1_OFF[a] + u * D1 + i];
#pragma unroll
                            for (int k = 0; k < D3; ++k) g[k] = s.tb[(l * TILE_R + r) * D3 + k];
                            sfor<CG_BEGIN[P], CG_BEGIN[P + 1]>([&](auto n_) {
                                constexpr int N = n_;
                                dy[CG_J[N]] = fma((T)CG_V[N] * g[CG_K[N]], x[CG_I[N]], dy[CG_J[N]]);
                            });
                        }
                    }
#pragma unroll
                    for (int j = 0; j < D2; ++j) {
                        const T sum = warp_sum(dy[j]);
                        if (lane == 0) s.gy[r * Y_DIM + IN2_OFF[b] + v * D2 + j] += sum;
                    }
                }
                __syncthreads();
            }
        });
        store_tile(p.dX, s.gx, row0, p.batch, X_DIM, tid);
        store_tile(p.dY, s.gy, row0, p.batch, Y_DIM, tid);
        __syncthreads();
    }
}

}  // namespace oeq

#define OEQ_K_UVW_FWD 10
#define OEQ_K_UVW_BWD 11

extern "C" __global__ void __launch_bounds__(oeq::NT, 1) oeq_uvw_kernel(const oeq::UvwParams p) {
#if OEQ_KERNEL == OEQ_K_UVW_FWD
    oeq::uvw_forward(p);
#elif OEQ_KERNEL == OEQ_K_UVW_BWD
    oeq::uvw_backward(p);
#else
#error "OEQ_KERNEL must select one of the uvw kernels"
#endif
}

// Fixed-order sum of the per-CTA partial weight gradients: dW[i] = sum_c ws[c][i].
extern "C" __global__ void oeq_reduce_partials(const oeqd::T* ws, oeqd::T* out, int n, long long groups) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    oeqd::T s = (oeqd::T)0;
    for (long long g = 0; g < groups; ++g) s += ws[g * n + i];
    out[i] = s;
}
