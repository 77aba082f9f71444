// Host runtime behind the C ABI (include/oeq_b200.h).
//
// Replaces the reference's native layer (openequivariance/extension/:
// JITTPImpl / JITConvImpl in tensorproducts.hpp:50-98 and convolution.hpp:94-176,
// the NVRTC + driver wrapper CUJITKernel in util/backend_cuda.hpp:139-300) and the
// launch-shape half of its scheduler (implementations/ComputationSchedule.py:232-425).
//
// For a problem it (1) picks the thread mapping (channels per group, path
// partitions, groups per CTA), (2) emits a small header of constexpr tables that
// describes the problem -- irreps, instructions, Clebsch-Gordan nonzeros scaled by
// the path weights, the mapping -- (3) compiles the hand-written kernel templates
// in csrc/*.cuh against it with NVRTC for sm_100a, caching the CUBIN on disk, and
// (4) launches through the CUDA runtime's library API on the caller's stream.
// No kernel body is generated; no CPU fallback exists.

#include <cuda_runtime.h>
#include <dlfcn.h>
#include <nvrtc.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <mutex>
#include <sstream>
#include <string>
#include <vector>

#include "../../include/oeq_b200.h"
#include "oeq_common.cuh"

namespace {

thread_local std::string g_error;
int fail(int code, const std::string& msg) {
    g_error = msg;
    return code;
}
#define OEQ_CUDA(expr)                                                                          \
    do {                                                                                        \
        cudaError_t e_ = (expr);                                                                \
        if (e_ != cudaSuccess)                                                                  \
            return fail(OEQ_ERR_CUDA, std::string(#expr) + ": " + cudaGetErrorString(e_));      \
    } while (0)

std::mutex g_mutex;
std::string g_kernel_dir, g_cache_dir;

std::string library_dir() {
    Dl_info info;
    if (dladdr(reinterpret_cast<void*>(&library_dir), &info) && info.dli_fname) {
        std::string p(info.dli_fname);
        size_t slash = p.find_last_of('/');
        return slash == std::string::npos ? std::string(".") : p.substr(0, slash);
    }
    return ".";
}
std::string kernel_dir() {
    if (!g_kernel_dir.empty()) return g_kernel_dir;
    if (const char* e = getenv("OEQ_B200_KERNEL_DIR")) return e;
    return library_dir() + "/csrc";
}
std::string cache_dir() {
    if (!g_cache_dir.empty()) return g_cache_dir;
    if (const char* e = getenv("OEQ_B200_CACHE_DIR")) return e;
    return library_dir() + "/_kcache";
}
int env_int(const char* name, int fallback) {
    const char* e = getenv(name);
    return e && *e ? atoi(e) : fallback;
}

// ------------------------------------------------------------------ NVRTC, loaded on first use

struct Nvrtc {
    void* lib = nullptr;
    decltype(&nvrtcCreateProgram) create = nullptr;
    decltype(&nvrtcCompileProgram) compile = nullptr;
    decltype(&nvrtcGetCUBINSize) cubin_size = nullptr;
    decltype(&nvrtcGetCUBIN) cubin = nullptr;
    decltype(&nvrtcGetProgramLogSize) log_size = nullptr;
    decltype(&nvrtcGetProgramLog) log = nullptr;
    decltype(&nvrtcDestroyProgram) destroy = nullptr;
    decltype(&nvrtcGetErrorString) error_string = nullptr;
};
Nvrtc g_nvrtc;

int load_nvrtc() {
    if (g_nvrtc.lib) return OEQ_OK;
    const char* names[] = {"libnvrtc.so.12", "/usr/local/cuda/lib64/libnvrtc.so.12", "libnvrtc.so",
                           "/usr/local/cuda/lib64/libnvrtc.so"};
    void* lib = nullptr;
    for (const char* n : names) {
        lib = dlopen(n, RTLD_NOW | RTLD_LOCAL);
        if (lib) break;
    }
    if (!lib) return fail(OEQ_ERR_COMPILE, "cannot load libnvrtc (needed to specialise kernels)");
#define OEQ_SYM(field, name)                                                      \
    g_nvrtc.field = reinterpret_cast<decltype(g_nvrtc.field)>(dlsym(lib, name));  \
    if (!g_nvrtc.field) return fail(OEQ_ERR_COMPILE, std::string("libnvrtc lacks ") + name);
    OEQ_SYM(create, "nvrtcCreateProgram")
    OEQ_SYM(compile, "nvrtcCompileProgram")
    OEQ_SYM(cubin_size, "nvrtcGetCUBINSize")
    OEQ_SYM(cubin, "nvrtcGetCUBIN")
    OEQ_SYM(log_size, "nvrtcGetProgramLogSize")
    OEQ_SYM(log, "nvrtcGetProgramLog")
    OEQ_SYM(destroy, "nvrtcDestroyProgram")
    OEQ_SYM(error_string, "nvrtcGetErrorString")
#undef OEQ_SYM
    g_nvrtc.lib = lib;
    return OEQ_OK;
}

// ------------------------------------------------------------------ problem model

struct Irrep {
    int mul, l, parity, dim, off;
};
struct Instr {
    int i1, i2, io, mode;
    double pw;
    std::vector<int> ci, cj, ck;
    std::vector<double> cv;
    int w_off;  // first weight of the instruction (same in e3nn and kernel order)
    long long cost() const { return (long long)cv.size(); }
};
struct Problem {
    std::vector<Irrep> in1, in2, out;
    std::vector<Instr> instr;
    int dtype = 0, shared = 0, mode = 0;
    int unit = 0;               // no weight array: every weight is 1 (shared_weights == 2 in the descriptor)
    int x_dim = 0, y_dim = 0, z_dim = 0, w_numel = 0;
    int elem() const { return dtype == OEQ_F64 ? 8 : 4; }
};

int ingest_irreps(const oeq_irrep* src, int n, std::vector<Irrep>& dst, int& dim, const char* what) {
    if (n < 0 || (n > 0 && !src)) return fail(OEQ_ERR_INVALID, std::string(what) + ": null irreps");
    int off = 0;
    for (int i = 0; i < n; ++i) {
        if (src[i].mul < 0 || src[i].l < 0 || (src[i].parity != 1 && src[i].parity != -1))
            return fail(OEQ_ERR_INVALID, std::string(what) + ": bad irrep entry");
        Irrep r{src[i].mul, src[i].l, src[i].parity, 2 * src[i].l + 1, off};
        off += r.mul * r.dim;
        dst.push_back(r);
    }
    dim = off;
    return OEQ_OK;
}

int ingest(const oeq_problem_desc* d, Problem& p) {
    if (!d) return fail(OEQ_ERR_INVALID, "null problem descriptor");
    if (d->dtype != OEQ_F32 && d->dtype != OEQ_F64) return fail(OEQ_ERR_INVALID, "dtype must be OEQ_F32 or OEQ_F64");
    p.dtype = d->dtype;
    p.unit = d->shared_weights == 2 ? 1 : 0;
    p.shared = (d->shared_weights && !p.unit) ? 1 : 0;
    int rc;
    if ((rc = ingest_irreps(d->in1, d->n_in1, p.in1, p.x_dim, "irreps_in1"))) return rc;
    if ((rc = ingest_irreps(d->in2, d->n_in2, p.in2, p.y_dim, "irreps_in2"))) return rc;
    if ((rc = ingest_irreps(d->out, d->n_out, p.out, p.z_dim, "irreps_out"))) return rc;
    if (d->n_instr <= 0 || !d->instr)
        return fail(OEQ_ERR_INVALID, "Tensor product problem has no valid intructions!");
    p.mode = d->instr[0].mode;
    if (p.mode != OEQ_MODE_UVU && p.mode != OEQ_MODE_UVW)
        return fail(OEQ_ERR_UNSUPPORTED, "connection mode must be 'uvu' or 'uvw'");
    int w = 0;
    for (int n = 0; n < d->n_instr; ++n) {
        const oeq_instruction& s = d->instr[n];
        if (s.mode != p.mode) return fail(OEQ_ERR_UNSUPPORTED, "all instructions must share one connection mode");
        if (s.i_in1 < 0 || s.i_in1 >= d->n_in1 || s.i_in2 < 0 || s.i_in2 >= d->n_in2 || s.i_out < 0 ||
            s.i_out >= d->n_out)
            return fail(OEQ_ERR_INVALID, "instruction index out of range");
        const Irrep &a = p.in1[s.i_in1], &b = p.in2[s.i_in2], &c = p.out[s.i_out];
        if (a.parity * b.parity != c.parity || c.l < std::abs(a.l - b.l) || c.l > a.l + b.l)
            return fail(OEQ_ERR_INVALID, "instruction violates the selection rules");
        if (p.mode == OEQ_MODE_UVU && a.mul != c.mul)
            return fail(OEQ_ERR_INVALID, "'uvu' needs equal multiplicities of the first input and the output");
        Instr t;
        t.i1 = s.i_in1; t.i2 = s.i_in2; t.io = s.i_out; t.mode = s.mode; t.pw = s.path_weight;
        if (s.cg_nnz < 0 || (s.cg_nnz > 0 && (!s.cg_i || !s.cg_j || !s.cg_k || !s.cg_value)))
            return fail(OEQ_ERR_INVALID, "instruction has a malformed Clebsch-Gordan list");
        for (int z = 0; z < s.cg_nnz; ++z) {
            if (s.cg_i[z] < 0 || s.cg_i[z] >= a.dim || s.cg_j[z] < 0 || s.cg_j[z] >= b.dim || s.cg_k[z] < 0 ||
                s.cg_k[z] >= c.dim)
                return fail(OEQ_ERR_INVALID, "Clebsch-Gordan index out of range");
            t.ci.push_back(s.cg_i[z]); t.cj.push_back(s.cg_j[z]); t.ck.push_back(s.cg_k[z]);
            t.cv.push_back(s.cg_value[z] * s.path_weight);
        }
        t.w_off = w;
        w += a.mul * b.mul * (p.mode == OEQ_MODE_UVW ? c.mul : 1);
        p.instr.push_back(std::move(t));
    }
    p.w_numel = w;
    return OEQ_OK;
}

// ------------------------------------------------------------------ thread mapping for the "uvu" kernels

enum Kind { K_FWD_BATCH = 0, K_BWD_BATCH, K_FWD_DET, K_BWD_DET, K_FWD_ATOMIC, K_BWD_ATOMIC, K_COUNT };
bool kind_is_bwd(int k) { return k & 1; }
bool kind_is_batch(int k) { return k < 2; }

constexpr int SMEM_LIMIT = 232448;  // opt-in dynamic shared memory per CTA on sm_100
int pad16(int b) { return (b + 15) / 16 * 16; }

struct Mapping {
    int mulg = 32, nch = 1, ps = 1, ng = 1, producer = 0, min_ctas = 1;
    int nph = 1;                              // backward staging in phases (see uvu_kernels.cuh)
    bool tc_tables = false;                   // emit the tables of the tensor-core forward pass
    std::vector<int> z_ph_begin, w_ph_begin;  // nph + 1 column / weight boundaries
    std::vector<int> phase_of_instr;
    std::vector<int> part_of_out, part_of_instr, zr_off, xr_off;
    int zpc_max = 1, xpc = 1;
    int stage_bytes = 0, extra_bytes = 0, sw_bytes = 0;
    int helper_warps = 0;                     // receiver-order backward: warps that sum the previous block's rows
    int gz_regs = 1 << 20, gz_smem_values = 0; // receiver-order backward: dZ values in registers / parked in shared memory
    int epi = 1;                              // edges per staged item (uvu_kernels.cuh, EPI)
    int stage_cap = 4;                        // most stages a group takes
    int chunk_floor = 32;                     // smallest chunk of consecutive edges a launch may deal out
    int threads() const { return ng * mulg * ps + 32 * ng * producer + 32 * helper_warps; }
    int fixed_bytes(int stages) const { return ng * stages * (16 + 8 * (epi > 1 ? 4 + 2 * epi : 4)) + ng * 128 + sw_bytes; }
    int smem(int stages) const { return fixed_bytes(stages) + ng * (stages * stage_bytes + extra_bytes); }
    int max_stages() const {
        int s = 0;
        while (s < stage_cap && smem(s + 1) <= SMEM_LIMIT) ++s;
        return s;
    }
};

void assign_partitions(const Problem& p, bool bwd, Mapping& m) {
    // longest-processing-time first; forward units are output irreps, backward units instructions
    const int n_units = bwd ? (int)p.instr.size() : (int)p.out.size();
    std::vector<long long> cost(n_units, 0);
    for (size_t i = 0; i < p.instr.size(); ++i) {
        long long c = p.instr[i].cost() * p.in2[p.instr[i].i2].mul + 2;
        cost[bwd ? (int)i : p.instr[i].io] += c;
    }
    std::vector<int> order(n_units);
    for (int i = 0; i < n_units; ++i) order[i] = i;
    std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return cost[a] > cost[b]; });
    std::vector<long long> load(m.ps, 0);
    std::vector<int> part(n_units, 0);
    for (int unit : order) {
        int best = 0;
        for (int q = 1; q < m.ps; ++q)
            if (load[q] < load[best]) best = q;
        part[unit] = best;
        load[best] += cost[unit];
    }
    m.part_of_out.assign(p.out.size(), 0);
    m.part_of_instr.assign(p.instr.size(), 0);
    if (bwd) {
        m.part_of_instr = part;
    } else {
        m.part_of_out = part;
        for (size_t i = 0; i < p.instr.size(); ++i) m.part_of_instr[i] = part[p.instr[i].io];
    }
    // register offsets of the per-channel accumulators
    m.zr_off.assign(p.out.size(), 0);
    std::vector<int> fill(m.ps, 0);
    for (size_t o = 0; o < p.out.size(); ++o) {
        int q = bwd ? 0 : m.part_of_out[o];
        m.zr_off[o] = fill[q];
        fill[q] += p.out[o].dim;
    }
    m.zpc_max = std::max(1, *std::max_element(fill.begin(), fill.end()));
    m.xr_off.assign(p.in1.size(), 0);
    int x = 0;
    for (size_t a = 0; a < p.in1.size(); ++a) {
        m.xr_off[a] = x;
        x += p.in1[a].dim;
    }
    m.xpc = std::max(1, x);
}

// Narrow self-staging groups (one warp per group) of the receiver-order walks stage runs of consecutive edges:
// the per-item fixed cost (list walk, copies, hand-off) is shared by up to `epi` edges.  Re-fits the group count.
void apply_edges_per_item(const Problem& p, Mapping& m, int extra_per_group) {
    m.epi = 1;
    const int want = env_int("OEQ_B200_EPI", 2);
    if (want <= 1 || want > 8 || m.producer || m.mulg * m.ps > 32 || p.shared) return;
    const int e = p.elem();
    const int xb = pad16(p.x_dim * e);
    const int wrow = p.unit ? 0 : p.w_numel * e;
    Mapping t = m;
    t.epi = want;
    t.stage_bytes = want * xb + pad16(want * p.y_dim * e) + pad16(want * wrow);
    t.extra_bytes = extra_per_group;
    // two stages of `want` edges keep as many edges in flight as four stages of one
    t.stage_cap = std::max(2, std::min(4, env_int("OEQ_B200_EPI_STAGES", 2)));
    while (t.ng > 1 && t.smem(t.stage_cap) > SMEM_LIMIT) --t.ng;
    if (t.smem(t.stage_cap) > SMEM_LIMIT) return;
    m = t;
    const int stages = std::min(m.max_stages(), env_int("OEQ_B200_STAGES", 4));
    const int by_smem = stages >= 2 ? SMEM_LIMIT / (m.smem(stages) + 1024) : 1;
    m.min_ctas = std::max(1, std::min({by_smem, 2048 / m.threads(), 2}));
}

int choose_mapping(const Problem& p, int kind, Mapping& m) {
    const bool bwd = kind_is_bwd(kind), batch = kind_is_batch(kind);
    int maxmul = 1;
    for (const Instr& t : p.instr) maxmul = std::max(maxmul, p.in1[t.i1].mul);
    for (const Irrep& r : p.out) maxmul = std::max(maxmul, r.mul);
    m.mulg = std::min((maxmul + 31) / 32 * 32, 256);
    m.nch = (maxmul + m.mulg - 1) / m.mulg;
    const int e = p.elem();
    const int xb = pad16(p.x_dim * e), yb = pad16(p.y_dim * e), zb = pad16(p.z_dim * e);
    const int wb = (p.shared || p.unit) ? 0 : pad16(p.w_numel * e);
    m.sw_bytes = p.shared ? pad16(p.w_numel * e) : 0;
    m.stage_bytes = xb + yb + wb + (bwd ? zb : 0);
    int zpc = 0;
    for (const Irrep& r : p.out) zpc += r.dim;
    const int units = bwd ? (int)p.instr.size() : (int)p.out.size();

    auto extra = [&](int ps) {
        const int warps = m.mulg * ps / 32;
        if (!bwd) return batch ? 2 * zb : 0;
        return ps * xb + 5 * warps * yb + (p.shared ? pad16(p.w_numel * e) : 0);
    };
    // Measured on B200: these kernels are bound by instruction issue, so the mapping that wins is the
    // one with the least per-thread overhead and the most independent groups per SM: one path
    // partition unless registers force more, and as many groups as shared memory admits.
    int xpc = 0;
    for (const Irrep& r : p.in1) xpc += r.dim;
    int best_ps = 1;
    if (!bwd) {
        auto regs = [&](int ps) { return zpc * m.nch / ps + xpc * m.nch + std::min(p.y_dim, 32) + 56; };
        while (regs(best_ps) > 232 && best_ps < 4 && best_ps * 2 <= units) best_ps *= 2;
    }
    auto groups_that_fit = [&](const Mapping& base, int ps) {
        Mapping t = base;
        t.ps = ps;
        t.extra_bytes = extra(ps);
        const int g = m.mulg * ps;
        const int want = std::max(1, std::min(8, (bwd ? 512 : (g >= 128 ? 128 : 256)) / g));
        for (int cand = want; cand >= 1; --cand) {
            t.ng = cand;
            if (t.smem(cand > 1 ? 2 : (bwd ? 2 : 3)) <= SMEM_LIMIT || (cand == 1 && t.smem(2) <= SMEM_LIMIT)) return cand;
        }
        return 0;
    };
    m.phase_of_instr.assign(p.instr.size(), 0);
    int best_ng = groups_that_fit(m, best_ps);
    m.nph = 1;
    m.z_ph_begin = {0, p.z_dim};
    m.w_ph_begin = {0, p.w_numel};
    const int max_phases = env_int("OEQ_B200_PHASES", 2);
    if (bwd && !batch && !p.shared) {
        // One or two groups per SM leave the issue slots half empty.  Stage the output-gradient row (the
        // bulk of a backward stage) in slices: cut the output irreps into nph runs of about equal width at
        // boundaries where the weights (ordered by instruction) split the same way; keep the largest
        // group count, preferring fewer phases.
        // (measured: going from one group to two pays; slicing further to reach three or four does not)
        const int target_groups = std::max(1, std::min(env_int("OEQ_B200_PHASE_GROUPS", 2), 512 / (m.mulg * best_ps)));
        for (int nph = 2; nph <= max_phases && best_ng < target_groups; ++nph) {
            std::vector<int> cut = {0};          // output irrep index where each phase starts
            for (int q = 1; q < nph; ++q) {
                const int want = (int)((long long)p.z_dim * q / nph);
                int best = -1;
                for (size_t os = cut.back() + 1; os < p.out.size(); ++os)
                    if (best < 0 || std::abs(p.out[os].off - want) < std::abs(p.out[best].off - want)) best = (int)os;
                if (best < 0) break;
                cut.push_back(best);
            }
            if ((int)cut.size() != nph) continue;
            cut.push_back((int)p.out.size());
            std::vector<int> zb(nph + 1), wbeg(nph + 1);
            bool ok = true;
            for (int q = 0; q <= nph; ++q) zb[q] = q == nph ? p.z_dim : p.out[cut[q]].off;
            // weights of phase q must be the contiguous run [wbeg[q], wbeg[q+1])
            wbeg[0] = 0;
            wbeg[nph] = p.w_numel;
            for (int q = 1; q < nph && ok; ++q) {
                int lo = p.w_numel;
                for (const Instr& t : p.instr)
                    if (t.io >= cut[q]) lo = std::min(lo, t.w_off);
                wbeg[q] = lo;
            }
            std::vector<int> phase(p.instr.size(), 0);
            for (size_t i = 0; i < p.instr.size() && ok; ++i) {
                const Instr& t = p.instr[i];
                int q = 0;
                while (q + 1 < nph && t.io >= cut[q + 1]) ++q;
                phase[i] = q;
                const int size = p.in1[t.i1].mul * p.in2[t.i2].mul;
                if (t.w_off < wbeg[q] || t.w_off + size > wbeg[q + 1]) ok = false;
            }
            for (int q = 0; q <= nph && ok; ++q)
                if ((zb[q] * e) % 16 || (wbeg[q] * e) % 16) ok = false;
            for (int q = 0; q < nph && ok; ++q)
                if (zb[q + 1] <= zb[q] || wbeg[q + 1] <= wbeg[q]) ok = false;
            if (!ok) continue;
            int wmax = 0, zmax = 0;
            for (int q = 0; q < nph; ++q) {
                wmax = std::max(wmax, wbeg[q + 1] - wbeg[q]);
                zmax = std::max(zmax, zb[q + 1] - zb[q]);
            }
            Mapping t = m;
            t.stage_bytes = xb + yb + (p.unit ? 0 : pad16(wmax * e)) + pad16(zmax * e);
            const int ng = groups_that_fit(t, best_ps);
            if (ng > best_ng) {
                best_ng = ng;
                m.stage_bytes = t.stage_bytes;
                m.nph = nph;
                m.z_ph_begin = zb;
                m.w_ph_begin = wbeg;
                m.phase_of_instr = phase;
            }
        }
    }
    if (best_ng == 0)
        return fail(OEQ_ERR_UNSUPPORTED, "problem rows do not fit in shared memory (two stages of one item exceed 227 KB)");
    m.ps = env_int(bwd ? "OEQ_B200_PS_BWD" : "OEQ_B200_PS_FWD", env_int("OEQ_B200_PS", best_ps));
    m.ng = env_int(bwd ? "OEQ_B200_NG_BWD" : "OEQ_B200_NG_FWD", env_int("OEQ_B200_NG", best_ng));
    m.extra_bytes = extra(m.ps);
    // a dedicated staging warp pays off for one wide group per CTA; many narrow groups stage their own items
    m.producer = env_int("OEQ_B200_PRODUCER", (m.ng <= 4 && m.mulg * m.ps >= 128) ? 1 : 0);
    if (m.ng > 4) m.producer = 0;
    {
        // let the compiler budget registers for as many CTAs per SM as shared memory admits
        const int stages = std::min(m.max_stages(), env_int("OEQ_B200_STAGES", 4));
        const int by_smem = stages >= 2 ? SMEM_LIMIT / (m.smem(stages) + 1024) : 1;
        const int by_threads = 2048 / m.threads();
        m.min_ctas = env_int("OEQ_B200_MIN_CTAS", std::max(1, std::min({by_smem, by_threads, 2})));
    }
    if (m.smem(2) > SMEM_LIMIT || m.ng * m.mulg * m.ps > 992 || m.ng < 1 || m.ng > 8)
        return fail(OEQ_ERR_INVALID, "OEQ_B200_PS / OEQ_B200_NG override does not fit");
    if (!bwd && !batch) apply_edges_per_item(p, m, m.extra_bytes);
    // deterministic walks align every chunk at a segment boundary (two dependent index reads per chunk)
    m.chunk_floor = (kind == K_FWD_DET || kind == K_BWD_DET) ? 64 : 32;
    assign_partitions(p, bwd, m);
    if (env_int("OEQ_B200_VERBOSE", 0))
        fprintf(stderr, "[oeq_b200] kind %d: mulg %d nch %d ps %d ng %d threads %d stage %d B extra %d B max stages %d\n",
                kind, m.mulg, m.nch, m.ps, m.ng, m.threads(), m.stage_bytes, m.extra_bytes, m.max_stages());
    return OEQ_OK;
}

// Receiver-order backward pass of the convolution (uvu_kernels.cuh, run_backward_recv): one thread per
// channel, stages as in the forward pass, two dX rows and the dY partials per group as extras.
constexpr int K_BWD_RECV_DET = 6, K_BWD_RECV_ATOMIC = 7;

bool recv_backward_supported(const Problem& p) {
    if (p.mode != OEQ_MODE_UVU || p.shared || p.y_dim > 32) return false;
    for (const Irrep& r : p.in2)
        if (r.mul != 1) return false;
    int maxmul = 1, zpc = 0, xpc = 0;
    for (const Instr& t : p.instr) maxmul = std::max(maxmul, p.in1[t.i1].mul);
    for (const Irrep& r : p.out) { maxmul = std::max(maxmul, r.mul); zpc += r.dim; }
    for (const Irrep& r : p.in1) xpc += r.dim;
    if (maxmul > 256) return false;                             // one thread per channel
    int d1max = 1;
    for (const Irrep& r : p.in1) d1max = std::max(d1max, r.dim);
    // the channel's slice of dZ lives in registers (32-bit registers: twice as many for FP64 values)
    if ((zpc + 2 * p.y_dim + 4 * d1max) * (p.elem() / 4) + 40 > 200) return false;
    return env_int("OEQ_B200_BWD_RECV", 1) != 0;
}

int choose_mapping_recv(const Problem& p, Mapping& m) {
    int maxmul = 1;
    for (const Instr& t : p.instr) maxmul = std::max(maxmul, p.in1[t.i1].mul);
    for (const Irrep& r : p.out) maxmul = std::max(maxmul, r.mul);
    m.mulg = (maxmul + 31) / 32 * 32;
    m.nch = 1;
    m.ps = 1;
    const int e = p.elem();
    const int xb = pad16(p.x_dim * e), yb = pad16(p.y_dim * e), wb = p.unit ? 0 : pad16(p.w_numel * e);
    m.sw_bytes = 0;
    m.stage_bytes = xb + yb + wb;
    // dZ values per channel beyond the register budget are parked in shared memory (whole output irreps)
    int zpc = 0;
    for (const Irrep& r : p.out) zpc += r.dim;
    const int budget = env_int("OEQ_B200_GZ_REGS", p.dtype == OEQ_F64 ? 28 : 56);
    m.gz_regs = budget;
    m.gz_smem_values = 0;
    {
        int off = 0;
        for (const Irrep& r : p.out) {
            if (off >= budget) m.gz_smem_values += r.dim;
            off += r.dim;
        }
    }
    m.extra_bytes = 2 * xb + 5 * (m.mulg / 32) * yb + pad16(m.gz_smem_values * m.mulg * e);
    m.nph = 1;
    m.z_ph_begin = {0, p.z_dim};
    m.w_ph_begin = {0, p.w_numel};
    m.phase_of_instr.assign(p.instr.size(), 0);
    // two wide groups share a CTA (one CTA per SM): 320 threads leave 200 registers per thread, which the
    // channel's dZ slice needs; two CTAs of 160 threads would be capped at 168
    const int want = std::max(1, std::min(8, 256 / m.mulg));
    m.ng = 0;
    for (int cand = want; cand >= 1 && !m.ng; --cand) {
        m.ng = cand;
        if (m.smem(cand > 1 ? 2 : 3) > SMEM_LIMIT && !(cand == 1 && m.smem(2) <= SMEM_LIMIT)) m.ng = 0;
    }
    if (!m.ng) return fail(OEQ_ERR_UNSUPPORTED, "problem rows do not fit in shared memory");
    m.ng = env_int("OEQ_B200_NG_RECV", m.ng);
    m.producer = env_int("OEQ_B200_PRODUCER", (m.ng <= 4 && m.mulg >= 128) ? 1 : 0);
    if (m.ng > 4) m.producer = 0;
    const int stages = std::min(m.max_stages(), env_int("OEQ_B200_STAGES", 4));
    const int by_smem = stages >= 2 ? SMEM_LIMIT / (m.smem(stages) + 1024) : 1;
    const int by_threads = 2048 / m.threads();
    m.min_ctas = env_int("OEQ_B200_MIN_CTAS_RECV", std::max(1, std::min({by_smem, by_threads, 2})));
    if (m.smem(2) > SMEM_LIMIT || m.ng < 1 || m.ng > 8) return fail(OEQ_ERR_INVALID, "OEQ_B200_NG_RECV override does not fit");
    apply_edges_per_item(p, m, m.extra_bytes);
    assign_partitions(p, true, m);
    if (env_int("OEQ_B200_VERBOSE", 0))
        fprintf(stderr, "[oeq_b200] receiver-order backward: mulg %d ng %d threads %d stage %d B extra %d B max stages %d min ctas %d\n",
                m.mulg, m.ng, m.threads(), m.stage_bytes, m.extra_bytes, m.max_stages(), m.min_ctas);
    return OEQ_OK;
}

// ------------------------------------------------------------------ descriptor text

template <class V, class F>
void emit_array(std::ostringstream& s, const char* type, const char* name, const V& v, F&& fmt) {
    s << "constexpr " << type << " " << name << "[] = {";
    if (v.empty()) s << "0";
    for (size_t i = 0; i < v.size(); ++i) {
        if (i) s << ", ";
        fmt(s, v[i]);
    }
    s << "};\n";
}

struct UvwConfig {
    int tile_r = 16, uvc = 64, dmax = 1, mwmax = 1, threads = 256;
    int smem(const Problem& p, bool bwd) const {
        auto r4 = [](long long n) { return (n + 3) / 4 * 4; };
        long long e = r4((long long)tile_r * p.x_dim) + r4((long long)tile_r * p.y_dim) + r4((long long)tile_r * p.z_dim) +
                      r4((long long)uvc * tile_r * dmax);
        if (bwd)
            e += r4((long long)tile_r * p.x_dim) + r4((long long)tile_r * p.y_dim) + r4((long long)mwmax * tile_r * dmax) +
                 r4((long long)uvc * tile_r * dmax);
        return (int)std::min<long long>(e * p.elem(), 1ll << 30);
    }
};

int choose_uvw(const Problem& p, bool bwd, UvwConfig& c) {
    for (const Irrep& r : p.out) {
        c.dmax = std::max(c.dmax, r.dim);
        c.mwmax = std::max(c.mwmax, r.mul);
    }
    int max_uv = 1;
    for (const Instr& t : p.instr) max_uv = std::max(max_uv, p.in1[t.i1].mul * p.in2[t.i2].mul);
    c.uvc = std::min(64, max_uv);
    for (int tile : {16, 8, 4}) {
        c.tile_r = tile;
        if (c.smem(p, bwd) <= SMEM_LIMIT) return OEQ_OK;
    }
    return fail(OEQ_ERR_UNSUPPORTED, "'uvw' problem rows do not fit in shared memory");
}

// ---- tensor-core forward pass of the 'uvu' convolution (mirrors the constexpr geometry of uvu_tc_kernels.cuh)
// Entry e of the per-edge matrix M[(p,k)][i] = sum_j c^p_ijk y_j: where it lives in the swizzled B tile and
// which (j, coefficient) terms it sums (dense [entry][tmax] table, coefficient 0 where an entry has fewer).
struct UvuTcTables {
    int n = 0, tmax = 1;
    std::vector<int> off, term_j;
    std::vector<double> term_c;
    int xpc = 0;
};

// Columns of the per-edge product: the paths of consumer partition q (the partition of their output
// irrep) are contiguous, in instruction order, and start at a multiple of 16.
struct UvuTcColumns {
    std::vector<int> col_begin;   // per instruction
    std::vector<int> part_col;    // per partition, plus the padded total
};

UvuTcColumns uvu_tc_columns(const Problem& p, const std::vector<int>& part_of_out, int parts) {
    UvuTcColumns c;
    c.col_begin.assign(p.instr.size(), 0);
    int cur = 0;
    for (int q = 0; q < parts; ++q) {
        cur = (cur + 15) / 16 * 16;
        c.part_col.push_back(cur);
        for (size_t i = 0; i < p.instr.size(); ++i)
            if (part_of_out[p.instr[i].io] == q) {
                c.col_begin[i] = cur;
                cur += p.out[p.instr[i].io].dim;
            }
    }
    c.part_col.push_back((cur + 15) / 16 * 16);
    return c;
}

int tc_swizzle_host(int row, int col) {
    return (row >> 3) * 1024 + (row & 7) * 128 + ((((col >> 2) ^ (row & 7)) & 7) << 4) + ((col & 3) << 2);
}

UvuTcTables build_uvu_tc_tables(const Problem& p, const UvuTcColumns& cols) {
    UvuTcTables t;
    std::vector<int> xoff(p.in1.size(), 0);
    for (size_t a = 0; a < p.in1.size(); ++a) {
        xoff[a] = t.xpc;
        t.xpc += p.in1[a].dim;
    }
    std::vector<std::vector<std::pair<int, double>>> terms;
    for (size_t pi = 0; pi < p.instr.size(); ++pi) {
        const Instr& ins = p.instr[pi];
        const int col0 = cols.col_begin[pi];
        const int d1 = p.in1[ins.i1].dim, d3 = p.out[ins.io].dim;
        for (int k = 0; k < d3; ++k)
            for (int i = 0; i < d1; ++i) {
                std::vector<std::pair<int, double>> tt;
                for (size_t z = 0; z < ins.ci.size(); ++z)
                    if (ins.ci[z] == i && ins.ck[z] == k) tt.push_back({p.in2[ins.i2].off + ins.cj[z], ins.cv[z]});
                if (tt.empty()) continue;
                t.off.push_back(tc_swizzle_host(col0 + k, xoff[ins.i1] + i));
                t.tmax = std::max(t.tmax, (int)tt.size());
                terms.push_back(std::move(tt));
            }
    }
    t.n = (int)t.off.size();
    t.term_j.assign((size_t)std::max(1, t.n) * t.tmax, 0);
    t.term_c.assign((size_t)std::max(1, t.n) * t.tmax, 0.0);
    for (int e = 0; e < t.n; ++e)
        for (size_t z = 0; z < terms[e].size(); ++z) {
            t.term_j[(size_t)e * t.tmax + z] = terms[e][z].first;
            t.term_c[(size_t)e * t.tmax + z] = terms[e][z].second;
        }
    if (t.off.empty()) t.off.push_back(0);
    return t;
}

struct UvuTcGeometry {
    int stages = 0, smem = 0;
};

// Problems the tensor-core forward pass takes: FP32 'uvu' with per-edge weights, second input of
// multiplicity 1 and at most 32 components, widest multiplicity 65..128 (thread = channel, M = 128 rows),
// at most 32 first-input components per channel (one swizzled 128-byte row) and 256 output columns.
bool uvu_tc_geometry(const Problem& p, UvuTcGeometry& g, int npad = 0) {
    if (p.mode != OEQ_MODE_UVU || p.shared || p.unit || p.dtype != OEQ_F32) return false;
    // Opt-in: measured on B200 the per-edge hand-offs between the roles make this kernel about twice as slow
    // as the FMA kernel (MACE-large, 1.5 M edges: 14.0 ms against 7.2 ms), so the FMA kernel is the default.
    if (!env_int("OEQ_B200_UVU_TC", 0)) return false;
    if (p.y_dim > 32) return false;
    int maxmul = 0, xpc = 0, ncols = 0;
    for (const Irrep& r : p.in1) {
        maxmul = std::max(maxmul, r.mul);
        xpc += r.dim;
    }
    for (const Instr& t : p.instr) {
        if (p.in2[t.i2].mul != 1) return false;
        ncols += p.out[t.io].dim;
    }
    if (maxmul <= 64 || maxmul > 128 || xpc > 32 || ncols > 224 || ncols == 0) return false;
    if ((p.x_dim * 4) % 16 || (p.w_numel * 4) % 16) return false;
    if (npad == 0) npad = (ncols + 15) / 16 * 16 + 16;      // upper bound: one padding gap between two partitions
    if (npad > 256) return false;
    const int off_stage = 2 * 2 * 128 * 128 + 2 * 2 * npad * 128 + 512;
    const int stage = pad16(p.x_dim * 4) + pad16(p.w_numel * 4) + pad16(p.y_dim * 4);
    g.stages = std::min(4, (SMEM_LIMIT - 1024 - off_stage) / stage);
    if (g.stages < 3) return false;
    g.smem = 1024 + off_stage + g.stages * stage;
    return true;
}

std::string descriptor_text(const Problem& p, const Mapping& m, const UvwConfig* uvw = nullptr) {
    std::ostringstream s;
    s.precision(17);
    s << "// problem descriptor (tables only; kernel bodies are in the included headers)\n";
    s << "namespace oeqd {\n";
    s << "typedef " << (p.dtype == OEQ_F64 ? "double" : "float") << " T;\n";
    s << "constexpr int X_DIM = " << p.x_dim << ", Y_DIM = " << p.y_dim << ", Z_DIM = " << p.z_dim
      << ", W_NUMEL = " << p.w_numel << ";\n";
    s << "constexpr bool SHARED_W = " << (p.shared ? "true" : "false") << ";\n";
    s << "constexpr bool UNIT_W = " << (p.unit ? "true" : "false") << ";\n";
    s << "constexpr int N_IN1 = " << p.in1.size() << ", N_IN2 = " << p.in2.size() << ", N_OUT = " << p.out.size()
      << ", N_INSTR = " << p.instr.size() << ";\n";
    auto put_int = [](std::ostringstream& o, int v) { o << v; };
    auto irreps = [&](const char* prefix, const std::vector<Irrep>& v) {
        std::vector<int> mul, dim, off;
        for (const Irrep& r : v) {
            mul.push_back(r.mul); dim.push_back(r.dim); off.push_back(r.off);
        }
        emit_array(s, "int", (std::string(prefix) + "_MUL").c_str(), mul, put_int);
        emit_array(s, "int", (std::string(prefix) + "_D").c_str(), dim, put_int);
        emit_array(s, "int", (std::string(prefix) + "_OFF").c_str(), off, put_int);
    };
    irreps("IN1", p.in1);
    irreps("IN2", p.in2);
    irreps("OUT", p.out);
    std::vector<int> i1, i2, io, woff, begin, ci, cj, ck;
    std::vector<double> cv;
    for (const Instr& t : p.instr) {
        i1.push_back(t.i1); i2.push_back(t.i2); io.push_back(t.io); woff.push_back(t.w_off);
        begin.push_back((int)ci.size());
        ci.insert(ci.end(), t.ci.begin(), t.ci.end());
        cj.insert(cj.end(), t.cj.begin(), t.cj.end());
        ck.insert(ck.end(), t.ck.begin(), t.ck.end());
        cv.insert(cv.end(), t.cv.begin(), t.cv.end());
    }
    begin.push_back((int)ci.size());
    emit_array(s, "int", "I_IN1", i1, put_int);
    emit_array(s, "int", "I_IN2", i2, put_int);
    emit_array(s, "int", "I_OUT", io, put_int);
    emit_array(s, "int", "W_OFF", woff, put_int);
    emit_array(s, "int", "CG_BEGIN", begin, put_int);
    emit_array(s, "int", "CG_I", ci, put_int);
    emit_array(s, "int", "CG_J", cj, put_int);
    emit_array(s, "int", "CG_K", ck, put_int);
    const bool f64 = p.dtype == OEQ_F64;
    emit_array(s, "T", "CG_V", cv, [f64](std::ostringstream& o, double v) {
        char buf[64];
        if (f64) snprintf(buf, sizeof buf, "%a", v);
        else snprintf(buf, sizeof buf, "%af", (double)(float)v);
        o << buf;
    });
    s << "constexpr int MULG = " << m.mulg << ", NCH = " << m.nch << ", PS = " << m.ps << ", NG = " << m.ng
      << ", PRODUCER = " << m.producer << ", MIN_CTAS = " << m.min_ctas << ", EPI = " << m.epi << ";\n";
    emit_array(s, "int", "FWD_PART_OF_OUT", m.part_of_out, put_int);
    emit_array(s, "int", "BWD_PART_OF_INSTR", m.part_of_instr, put_int);
    emit_array(s, "int", "ZR_OFF", m.zr_off, put_int);
    emit_array(s, "int", "XR_OFF", m.xr_off, put_int);
    {
        std::vector<int> ph = m.phase_of_instr;
        ph.resize(p.instr.size(), 0);
        emit_array(s, "int", "BWD_PHASE_OF_INSTR", ph, put_int);
        s << "constexpr int BWD_NPH = " << m.nph << ";\n";
        std::vector<int> zb = m.z_ph_begin, wb2 = m.w_ph_begin;
        if (zb.empty()) zb = {0, p.z_dim};
        if (wb2.empty()) wb2 = {0, p.w_numel};
        emit_array(s, "int", "Z_PH_BEGIN", zb, put_int);
        emit_array(s, "int", "W_PH_BEGIN", wb2, put_int);
        // the same tables again with device storage, for run-time indexing by phase
        s << "__device__ const int Z_PH_BEGIN_DEV[] = {";
        for (size_t i = 0; i < zb.size(); ++i) s << (i ? ", " : "") << zb[i];
        s << "};\n__device__ const int W_PH_BEGIN_DEV[] = {";
        for (size_t i = 0; i < wb2.size(); ++i) s << (i ? ", " : "") << wb2[i];
        s << "};\n";
    }
    s << "constexpr int ZPC_MAX = " << m.zpc_max << ", XPC = " << m.xpc << ";\n";
    s << "constexpr int GZ_REGS = " << m.gz_regs << ", GZ_SMEM_VALUES = " << m.gz_smem_values << ";\n";
    // cycle accounting inside the kernels is a development aid: it exists only in a library built with
    // -DOEQ_DEV_PROFILE (the shipped entry points then contain no allocation, synchronisation or printing)
#ifdef OEQ_DEV_PROFILE
    s << "constexpr bool UVU_PROFILE = " << (env_int("OEQ_B200_UVU_PROFILE", 0) ? "true" : "false") << ";\n";
#else
    s << "constexpr bool UVU_PROFILE = false;\n";
#endif
    if (m.tc_tables) {
        const UvuTcColumns cols = uvu_tc_columns(p, m.part_of_out, m.ps);
        const UvuTcTables t = build_uvu_tc_tables(p, cols);
        emit_array(s, "int", "TC_COL_BEGIN", cols.col_begin, put_int);
        emit_array(s, "int", "TC_PART_COL", cols.part_col, put_int);
        s << "constexpr int TCM_N = " << t.n << ", TCM_TMAX = " << t.tmax << ";\n";
        auto dev_ints = [&](const char* name, const std::vector<int>& v) {
            s << "__device__ const int " << name << "[] = {";
            for (size_t i = 0; i < v.size(); ++i) s << (i ? ", " : "") << v[i];
            s << "};\n";
        };
        dev_ints("TCM_OFF_DEV", t.off);
        dev_ints("TCM_J_DEV", t.term_j);
        s << "__device__ const float TCM_C_DEV[] = {";
        for (size_t i = 0; i < t.term_c.size(); ++i) {
            char buf[64];
            snprintf(buf, sizeof buf, "%af", (double)(float)t.term_c[i]);
            s << (i ? ", " : "") << buf;
        }
        s << "};\n";
    }
    if (uvw)
        s << "constexpr int TILE_R = " << uvw->tile_r << ", UVC = " << uvw->uvc << ", DMAX = " << uvw->dmax
          << ", MWMAX = " << uvw->mwmax << ", UVW_THREADS = " << uvw->threads << ";\n";
    s << "}  // namespace oeqd\n";
    return s.str();
}

// ------------------------------------------------------------------ compile + cache

unsigned long long fnv1a(const std::string& s, unsigned long long h = 1469598103934665603ull) {
    for (unsigned char c : s) {
        h ^= c;
        h *= 1099511628211ull;
    }
    return h;
}

bool read_file(const std::string& path, std::string& out) {
    std::ifstream f(path, std::ios::binary);
    if (!f) return false;
    std::ostringstream ss;
    ss << f.rdbuf();
    out = ss.str();
    return true;
}

struct Compiled {
    std::string cubin;
    std::string log;
};

int compile_kernel(const std::string& descriptor, const std::string& main_header, int kernel_id, Compiled& out) {
    std::lock_guard<std::mutex> lock(g_mutex);
    const std::string dir = kernel_dir();
    std::string common, body;
    if (!read_file(dir + "/oeq_common.cuh", common) || !read_file(dir + "/" + main_header, body))
        return fail(OEQ_ERR_COMPILE, "kernel headers not found in " + dir);
    for (const char* inc : {"tc_common.cuh", "uvu_kernels.cuh"}) {   // headers that the kernel files include
        std::string text;
        if (main_header != inc && read_file(dir + "/" + inc, text)) common += text;
    }
    const std::string source = descriptor + "#define OEQ_KERNEL " + std::to_string(kernel_id) + "\n#include \"" +
                               main_header + "\"\n";
    const std::string options = "-arch=sm_100a -std=c++17 -lineinfo -default-device -diag-suppress 177";
    unsigned long long h = fnv1a(source);
    h = fnv1a(common, h);
    h = fnv1a(body, h);
    h = fnv1a(options, h);
    char name[64];
    snprintf(name, sizeof name, "/k_%016llx.cubin", h);
    const std::string cdir = cache_dir();
    const std::string path = cdir + name;
    if (!env_int("OEQ_B200_NO_CACHE", 0) && read_file(path, out.cubin) && !out.cubin.empty()) return OEQ_OK;

    int rc = load_nvrtc();
    if (rc) return rc;
    nvrtcProgram prog;
    if (g_nvrtc.create(&prog, source.c_str(), "oeq_specialisation.cu", 0, nullptr, nullptr) != NVRTC_SUCCESS)
        return fail(OEQ_ERR_COMPILE, "nvrtcCreateProgram failed");
    const std::string inc = "-I" + dir;
    std::vector<const char*> opts = {"-arch=sm_100a", "-std=c++17", "-lineinfo", "-default-device", "-diag-suppress=177", inc.c_str()};
    std::string ptxas_v = "--ptxas-options=-v";
    if (env_int("OEQ_B200_VERBOSE", 0)) opts.push_back(ptxas_v.c_str());
    std::string maxreg = "--maxrregcount=" + std::to_string(env_int("OEQ_B200_MAXRREG", 0));
    if (env_int("OEQ_B200_MAXRREG", 0) > 0) opts.push_back(maxreg.c_str());
    nvrtcResult res = g_nvrtc.compile(prog, (int)opts.size(), opts.data());
    size_t log_size = 0;
    g_nvrtc.log_size(prog, &log_size);
    out.log.assign(log_size, '\0');
    if (log_size > 1) g_nvrtc.log(prog, &out.log[0]);
    if (env_int("OEQ_B200_VERBOSE", 0) && log_size > 1) fprintf(stderr, "[oeq_b200] %s\n", out.log.c_str());
    if (res != NVRTC_SUCCESS) {
        g_nvrtc.destroy(&prog);
        if (env_int("OEQ_B200_KEEP_SOURCE", 0)) {
            std::ofstream f("/tmp/oeq_failed_specialisation.cu");
            f << source;
        }
        return fail(OEQ_ERR_COMPILE, std::string("kernel specialisation failed: ") + g_nvrtc.error_string(res) + "\n" +
                                         out.log.substr(0, 4000));
    }
    size_t size = 0;
    g_nvrtc.cubin_size(prog, &size);
    out.cubin.assign(size, '\0');
    g_nvrtc.cubin(prog, &out.cubin[0]);
    g_nvrtc.destroy(&prog);
    mkdir(cdir.c_str(), 0755);
    const std::string tmp = path + ".tmp" + std::to_string((long long)getpid());
    {
        std::ofstream f(tmp, std::ios::binary);
        f.write(out.cubin.data(), (std::streamsize)out.cubin.size());
    }
    rename(tmp.c_str(), path.c_str());
    return OEQ_OK;
}

// ------------------------------------------------------------------ a specialised kernel

struct Kernel {
    Mapping map;
    UvwConfig uvw;
    bool is_uvw = false;
    Compiled code;
    bool compiled = false, loaded = false;
    cudaLibrary_t lib = nullptr;
    cudaKernel_t fn = nullptr, reduce_fn = nullptr;
    int stages = 0, smem = 0, regs = 0, ctas_per_sm = 1, sm_count = 0;
    bool is_uvu_tc = false;       // tensor-core forward of the convolution: one CTA per SM
    UvuTcGeometry tc_geo;
    int threads() const { return is_uvu_tc ? 128 * map.ps + 64 : map.threads(); }
};

int build_uvu(const Problem& p, int kind, Kernel& k) {
    int rc = choose_mapping(p, kind, k.map);
    if (rc) return rc;
    rc = compile_kernel(descriptor_text(p, k.map), "uvu_kernels.cuh", kind, k.code);
    if (rc) return rc;
    k.compiled = true;
    return OEQ_OK;
}

// One-pass second derivatives of the batch 'uvu' product (uvu_kernels.cuh, run_double_backward): per-row
// weights, second input of multiplicity 1 with at most 32 components, at most 256 channels; a row's seven
// arrays form one stage.
constexpr int K_DBL_BATCH = 8;

bool double_backward_supported(const Problem& p) {
    if (p.mode != OEQ_MODE_UVU || p.shared || p.unit || p.y_dim > 32) return false;
    for (const Irrep& r : p.in2)
        if (r.mul != 1) return false;
    int maxmul = 1, zpc = 0, d1max = 1;
    for (const Instr& t : p.instr) maxmul = std::max(maxmul, p.in1[t.i1].mul);
    for (const Irrep& r : p.out) { maxmul = std::max(maxmul, r.mul); zpc += r.dim; }
    for (const Irrep& r : p.in1) d1max = std::max(d1max, r.dim);
    if (maxmul > 256) return false;
    if ((zpc + 3 * p.y_dim + 5 * d1max) * (p.elem() / 4) + 40 > 232) return false;   // registers per thread
    return env_int("OEQ_B200_FUSED_DOUBLE_BACKWARD", 1) != 0;
}

int build_uvu_dbl(const Problem& p, Kernel& k) {
    Mapping& m = k.map;
    int maxmul = 1;
    for (const Instr& t : p.instr) maxmul = std::max(maxmul, p.in1[t.i1].mul);
    for (const Irrep& r : p.out) maxmul = std::max(maxmul, r.mul);
    m.mulg = (maxmul + 31) / 32 * 32;
    m.nch = 1; m.ps = 1; m.producer = 1;
    const int e = p.elem();
    const int xb = pad16(p.x_dim * e), yb = pad16(p.y_dim * e), wb = pad16(p.w_numel * e), zb = pad16(p.z_dim * e);
    m.sw_bytes = 0;
    m.stage_bytes = 2 * xb + 2 * yb + 2 * wb + zb;
    m.extra_bytes = 5 * (m.mulg / 32) * yb;
    m.nph = 1;
    m.z_ph_begin = {0, p.z_dim};
    m.w_ph_begin = {0, p.w_numel};
    m.phase_of_instr.assign(p.instr.size(), 0);
    m.ng = 0;
    for (int cand = std::max(1, std::min(4, 256 / m.mulg)); cand >= 1 && !m.ng; --cand) {
        m.ng = cand;
        if (m.smem(2) > SMEM_LIMIT) m.ng = 0;
    }
    if (!m.ng) return fail(OEQ_ERR_UNSUPPORTED, "a row's seven arrays do not fit two shared-memory stages");
    const int stages = std::min(m.max_stages(), 4);
    m.min_ctas = std::max(1, std::min({stages >= 2 ? SMEM_LIMIT / (m.smem(stages) + 1024) : 1, 2048 / m.threads(), 2}));
    assign_partitions(p, true, m);
    int rc = compile_kernel(descriptor_text(p, m), "uvu_kernels.cuh", K_DBL_BATCH, k.code);
    if (rc) return rc;
    k.compiled = true;
    return OEQ_OK;
}

int build_uvu_recv(const Problem& p, bool deterministic, Kernel& k) {
    int rc = choose_mapping_recv(p, k.map);
    if (rc) return rc;
    // Deterministic variant: two helper warps per CTA sum the previous block's dX rows while the consumers
    // work.  With two wide groups and their staging warps that makes twelve warps, three per scheduler, the
    // same register ceiling (168) as the ten warps without helpers.
    k.map.helper_warps = deterministic ? std::max(0, env_int("OEQ_B200_HELPER_WARPS", 2)) : 0;
    // narrow problems: their launches are too short for the pipelined row sum, and the two extra warps would
    // lower the register ceiling of the one-warp groups
    if (k.map.threads() > 1024 || k.map.epi > 1) k.map.helper_warps = 0;
    k.map.chunk_floor = deterministic ? 64 : 32;
    const std::string macros = "#define OEQ_HELPER_WARPS " + std::to_string(k.map.helper_warps) + "\n";
    rc = compile_kernel(descriptor_text(p, k.map) + macros, "uvu_kernels.cuh", deterministic ? K_BWD_RECV_DET : K_BWD_RECV_ATOMIC, k.code);
    if (rc) return rc;
    k.compiled = true;
    return OEQ_OK;
}

// Second derivatives of the convolution in two launches (uvu_kernels.cuh, DBLC): a forward-like walk for the
// gradient with respect to dZ and a receiver-order walk for the gradients with respect to X, Y, W.  Stages
// carry the cotangent rows next to X, Y, W.
constexpr int K_DBLC_Z_DET = 40, K_DBLC_Z_ATOMIC = 41, K_DBLC_G_DET = 42, K_DBLC_G_ATOMIC = 43;

bool conv_double_backward_supported(const Problem& p) {
    if (p.unit || !recv_backward_supported(p)) return false;
    int zpc = 0, xpc = 0;
    for (const Irrep& r : p.out) zpc += r.dim;
    for (const Irrep& r : p.in1) xpc += r.dim;
    if ((zpc + 3 * xpc + 2 * p.y_dim) * (p.elem() / 4) + 48 > 240) return false;    // registers of the forward-like walk
    return env_int("OEQ_B200_FUSED_DOUBLE_BACKWARD", 1) != 0;
}

int build_uvu_dblc(const Problem& p, bool deterministic, bool grads, Kernel& k) {
    Mapping& m = k.map;
    const int e = p.elem();
    const int xb = pad16(p.x_dim * e), yb = pad16(p.y_dim * e), wb = pad16(p.w_numel * e);
    int rc;
    if (grads) {
        if ((rc = choose_mapping_recv(p, m))) return rc;
        m.epi = 1;
        m.stage_cap = 4;
        // fewer dZ values in registers than the first-derivative pass: the cotangents take their place
        const int budget = env_int("OEQ_B200_GZ_REGS_DBL", p.dtype == OEQ_F64 ? 14 : 32);
        m.gz_regs = budget;
        m.gz_smem_values = 0;
        int off = 0;
        for (const Irrep& r : p.out) {
            if (off >= budget) m.gz_smem_values += r.dim;
            off += r.dim;
        }
        m.extra_bytes = 2 * xb + 5 * (m.mulg / 32) * yb + pad16(m.gz_smem_values * m.mulg * e);
    } else {
        int maxmul = 1;
        for (const Instr& t : p.instr) maxmul = std::max(maxmul, p.in1[t.i1].mul);
        for (const Irrep& r : p.out) maxmul = std::max(maxmul, r.mul);
        m.mulg = (maxmul + 31) / 32 * 32;
        m.nch = 1; m.ps = 1;
        m.sw_bytes = 0;
        m.extra_bytes = 0;
        m.nph = 1;
        m.z_ph_begin = {0, p.z_dim};
        m.w_ph_begin = {0, p.w_numel};
        m.phase_of_instr.assign(p.instr.size(), 0);
    }
    m.helper_warps = 0;
    m.stage_bytes = 2 * (xb + yb + wb);
    m.ng = 0;
    for (int cand = std::max(1, std::min(8, 256 / m.mulg)); cand >= 1 && !m.ng; --cand) {
        m.ng = cand;
        if (m.smem(2) > SMEM_LIMIT) m.ng = 0;
    }
    if (!m.ng) return fail(OEQ_ERR_UNSUPPORTED, "an edge's rows and cotangent rows do not fit two shared-memory stages");
    m.producer = (m.ng <= 4 && m.mulg >= 128) ? 1 : 0;
    const int stages = std::min(m.max_stages(), 4);
    m.min_ctas = std::max(1, std::min({stages >= 2 ? SMEM_LIMIT / (m.smem(stages) + 1024) : 1, 2048 / m.threads(), 2}));
    assign_partitions(p, grads, m);
    const int kind = grads ? (deterministic ? K_DBLC_G_DET : K_DBLC_G_ATOMIC) : (deterministic ? K_DBLC_Z_DET : K_DBLC_Z_ATOMIC);
    const std::string macros = "#define OEQ_HELPER_WARPS 0\n";
    rc = compile_kernel(descriptor_text(p, m) + macros, "uvu_kernels.cuh", kind, k.code);
    if (rc) return rc;
    k.compiled = true;
    return OEQ_OK;
}

constexpr int K_FWD_DET_TC = 30, K_FWD_ATOMIC_TC = 31;

int build_uvu_tc(const Problem& p, bool deterministic, Kernel& k) {
    if (!uvu_tc_geometry(p, k.tc_geo)) return fail(OEQ_ERR_UNSUPPORTED, "problem does not qualify for the tensor-core forward pass");
    Mapping& m = k.map;
    m.mulg = 128; m.nch = 1; m.ng = 1; m.producer = 1; m.min_ctas = 1;
    m.ps = std::max(1, std::min({2, (int)p.out.size(), env_int("OEQ_B200_TC_PARTS", 2)}));
    m.z_ph_begin = {0, p.z_dim};
    m.w_ph_begin = {0, p.w_numel};
    m.phase_of_instr.assign(p.instr.size(), 0);
    m.tc_tables = true;
    assign_partitions(p, false, m);
    const UvuTcColumns cols = uvu_tc_columns(p, m.part_of_out, m.ps);
    if (!uvu_tc_geometry(p, k.tc_geo, cols.part_col.back()))
        return fail(OEQ_ERR_UNSUPPORTED, "problem does not fit the tensor-core forward pass");
    k.is_uvu_tc = true;
    int rc = compile_kernel(descriptor_text(p, m), "uvu_tc_kernels.cuh", deterministic ? K_FWD_DET_TC : K_FWD_ATOMIC_TC, k.code);
    if (rc) return rc;
    k.compiled = true;
    return OEQ_OK;
}

constexpr int K_UVW_FWD = 10, K_UVW_BWD = 11;

int build_uvw(const Problem& p, int kind, Kernel& k) {
    k.is_uvw = true;
    int rc = choose_uvw(p, kind == K_UVW_BWD, k.uvw);
    if (rc) return rc;
    // the uvu mapping tables are emitted with neutral values so that one descriptor format serves both
    k.map.part_of_out.assign(p.out.size(), 0);
    k.map.part_of_instr.assign(p.instr.size(), 0);
    k.map.zr_off.assign(p.out.size(), 0);
    k.map.xr_off.assign(p.in1.size(), 0);
    rc = compile_kernel(descriptor_text(p, k.map, &k.uvw), "uvw_kernels.cuh", kind, k.code);
    if (rc) return rc;
    k.compiled = true;
    return OEQ_OK;
}

// ---- tensor-core forward for 'uvw' (mirrors the constexpr geometry of uvw_tc_kernels.cuh)
constexpr int K_UVW_TC_FWD = 20;

struct TcGeometry {
    size_t packed_bytes = 0;
    int smem = 0;
};

bool uvw_tc_geometry(const Problem& p, TcGeometry& g) {
    if (p.mode != OEQ_MODE_UVW || !p.shared || p.dtype != OEQ_F32) return false;
    if (!env_int("OEQ_B200_UVW_TC", 1)) return false;
    int w_max = 0, mw_max = 16;
    size_t total = 0;
    for (size_t o = 0; o < p.out.size(); ++o) {
        int blocks = 0;
        for (const Instr& t : p.instr)
            if (t.io == (int)o) {
                if (p.in2[t.i2].mul != 1) return false;
                blocks += (p.in1[t.i1].mul + 31) / 32;
            }
        if (blocks == 0) continue;
        const int mw = p.out[o].mul;
        if (mw % 16 != 0 || mw > 256 || p.out[o].dim > 64) return false;
        const int bytes = blocks * 2 * mw * 128;
        w_max = std::max(w_max, bytes);
        mw_max = std::max(mw_max, mw);
        total += bytes;
    }
    if (total == 0) return false;
    const int off_w = 2 * 2 * 128 * 128;
    const int off_stg = off_w + (w_max + 1023) / 1024 * 1024;
    const int off_bar = off_stg + (128 * (mw_max + 1) * 4 + 15) / 16 * 16;
    g.smem = off_bar + (2 * 2 + 2 * 32 + 2) * 8 + 16 + 1024;
    g.packed_bytes = total;
    return g.smem <= SMEM_LIMIT;
}

int build_uvw_tc(const Problem& p, Kernel& k) {
    k.is_uvw = true;
    int rc = choose_uvw(p, false, k.uvw);
    if (rc) return rc;
    k.map.part_of_out.assign(p.out.size(), 0);
    k.map.part_of_instr.assign(p.instr.size(), 0);
    k.map.zr_off.assign(p.out.size(), 0);
    k.map.xr_off.assign(p.in1.size(), 0);
    rc = compile_kernel(descriptor_text(p, k.map, &k.uvw), "uvw_tc_kernels.cuh", K_UVW_TC_FWD, k.code);
    if (rc) return rc;
    k.compiled = true;
    return OEQ_OK;
}

// ---- tensor-core backward for 'uvw' (mirrors the constexpr geometry of uvw_tc_bwd_kernels.cuh)
constexpr int K_UVW_TC_DW = 21, K_UVW_TC_DXY = 22;

struct TcBwdGeometry {
    int dw_smem = 0;
    int dxy_smem = 0;           // 0: the dX/dY kernel does not take this problem
    size_t wt_bytes = 0;        // transposed packed weights
};

bool uvw_tc_bwd_geometry(const Problem& p, TcBwdGeometry& g) {
    TcGeometry fwd;
    if (!uvw_tc_geometry(p, fwd)) return false;          // same class of problems as the forward pass
    if (!env_int("OEQ_B200_UVW_TC_BWD", 1)) return false;
    int mw_max = 16;
    for (const Irrep& r : p.out) mw_max = std::max(mw_max, r.mul);
    for (const Instr& t : p.instr)
        if (p.in1[t.i1].mul > 128) return false;
    if (mw_max > 128) return false;
    const int stage = 2 * 128 * 128 + 2 * mw_max * 128;
    const int stages = std::min(4, (200 * 1024) / stage);
    if (stages < 2) return false;
    g.dw_smem = stages * stage + (2 * stages + 4) * 8 + 16 + 1024;
    if (g.dw_smem > SMEM_LIMIT) return false;
    // dX/dY kernel: one set of A tiles, two buffers of one path's transposed weights, the epilogue staging
    // buffer, two sets of an X row and a dX row per epilogue warp
    int kb_max = 1, mup_max = 16, wt_max = 0, row_max = 0;
    size_t wt_total = 0;
    for (const Irrep& r : p.out) kb_max = std::max(kb_max, (r.mul + 31) / 32);
    for (const Instr& t : p.instr) {
        const int mup = (p.in1[t.i1].mul + 15) / 16 * 16;
        const int bytes = ((p.out[t.io].mul + 31) / 32) * 2 * mup * 128;
        mup_max = std::max(mup_max, mup);
        wt_max = std::max(wt_max, bytes);
        wt_total += bytes;
        row_max = std::max(row_max, p.in1[t.i1].mul * p.in1[t.i1].dim);
    }
    const int nacc = std::min(4, 512 / (2 * mup_max));
    const int off_w = kb_max * 2 * 128 * 128;
    const int off_stg = off_w + 2 * ((wt_max + 1023) / 1024 * 1024);
    const int off_row = off_stg + (128 * (mup_max + 1) * 4 + 15) / 16 * 16;
    const int off_bar = off_row + 12 * 4 * ((row_max * 4 + 15) / 16 * 16);
    const int dxy = off_bar + (2 * 1 + 2 * nacc + 4) * 8 + 16 + 1024;
    if (nacc >= 1 && dxy <= SMEM_LIMIT) {
        g.dxy_smem = dxy;
        g.wt_bytes = wt_total;
    }
    return true;
}

int build_uvw_tc_bwd(const Problem& p, int kernel_id, Kernel& k) {
    k.is_uvw = true;
    int rc = choose_uvw(p, true, k.uvw);
    if (rc) return rc;
    k.map.part_of_out.assign(p.out.size(), 0);
    k.map.part_of_instr.assign(p.instr.size(), 0);
    k.map.zr_off.assign(p.out.size(), 0);
    k.map.xr_off.assign(p.in1.size(), 0);
    rc = compile_kernel(descriptor_text(p, k.map, &k.uvw), "uvw_tc_bwd_kernels.cuh", kernel_id, k.code);
    if (rc) return rc;
    k.compiled = true;
    return OEQ_OK;
}

int build_tp(const Problem& p, bool bwd, Kernel& k) {
    if (p.mode == OEQ_MODE_UVW) return build_uvw(p, bwd ? K_UVW_BWD : K_UVW_FWD, k);
    return build_uvu(p, bwd ? K_BWD_BATCH : K_FWD_BATCH, k);
}

int load_uvw(Kernel& k, const Problem& p, bool bwd) {
    if (k.loaded) return OEQ_OK;
    OEQ_CUDA(cudaLibraryLoadData(&k.lib, k.code.cubin.data(), nullptr, nullptr, 0, nullptr, nullptr, 0));
    OEQ_CUDA(cudaLibraryGetKernel(&k.fn, k.lib, "oeq_uvw_kernel"));
    OEQ_CUDA(cudaLibraryGetKernel(&k.reduce_fn, k.lib, "oeq_reduce_partials"));
    int dev = 0;
    OEQ_CUDA(cudaGetDevice(&dev));
    OEQ_CUDA(cudaDeviceGetAttribute(&k.sm_count, cudaDevAttrMultiProcessorCount, dev));
    k.smem = k.uvw.smem(p, bwd);
    OEQ_CUDA(cudaFuncSetAttribute((const void*)k.fn, cudaFuncAttributeMaxDynamicSharedMemorySize, k.smem));
    cudaFuncAttributes attr;
    if (cudaFuncGetAttributes(&attr, (const void*)k.fn) == cudaSuccess) k.regs = attr.numRegs;
    else (void)cudaGetLastError();
    int occ = 1;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, (const void*)k.fn, k.uvw.threads, k.smem) != cudaSuccess) {
        (void)cudaGetLastError();
        occ = 1;
    }
    k.ctas_per_sm = std::max(1, std::min(occ, 2));
    k.map.ng = 1;
    k.loaded = true;
    return OEQ_OK;
}

// Mirror of oeq::UvwParams (uvw_kernels.cuh).
struct UvwParams {
    const void* X; const void* Y; const void* W; void* Z;
    const void* dZ; void* dX; void* dY; void* dW;
    void* ws;
    long long batch;
    int* status;
    int skip_dw;      // the shared-weight gradient comes from the tensor-core kernel
};

long long uvw_grid(const Kernel& k, long long batch) {
    const long long tiles = (batch + k.uvw.tile_r - 1) / k.uvw.tile_r;
    return std::max<long long>(1, std::min<long long>((long long)k.sm_count * k.ctas_per_sm, tiles));
}

int load_kernel(Kernel& k, const char* entry, bool want_reduce) {
    if (k.loaded) return OEQ_OK;
    OEQ_CUDA(cudaLibraryLoadData(&k.lib, k.code.cubin.data(), nullptr, nullptr, 0, nullptr, nullptr, 0));
    OEQ_CUDA(cudaLibraryGetKernel(&k.fn, k.lib, entry));
    if (want_reduce) OEQ_CUDA(cudaLibraryGetKernel(&k.reduce_fn, k.lib, "oeq_reduce_partials"));
    int dev = 0;
    OEQ_CUDA(cudaGetDevice(&dev));
    OEQ_CUDA(cudaDeviceGetAttribute(&k.sm_count, cudaDevAttrMultiProcessorCount, dev));
    int stages = std::min(k.map.max_stages(), env_int("OEQ_B200_STAGES", 4));
    if (k.is_uvu_tc) stages = k.tc_geo.stages;
    if (stages < 2) return fail(OEQ_ERR_UNSUPPORTED, "not enough shared memory for two stages");
    k.stages = stages;
    k.smem = k.is_uvu_tc ? k.tc_geo.smem : k.map.smem(stages);
    OEQ_CUDA(cudaFuncSetAttribute((const void*)k.fn, cudaFuncAttributeMaxDynamicSharedMemorySize, k.smem));
    cudaFuncAttributes attr;
    if (cudaFuncGetAttributes(&attr, (const void*)k.fn) == cudaSuccess) k.regs = attr.numRegs;
    else (void)cudaGetLastError();
    int occ = 1;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, (const void*)k.fn, k.threads(), k.smem) != cudaSuccess) {
        (void)cudaGetLastError();
        occ = 1;
    }
    k.ctas_per_sm = std::max(1, std::min(occ, env_int("OEQ_B200_CTAS_PER_SM", 4)));
    if (k.is_uvu_tc) k.ctas_per_sm = 1;
    k.loaded = true;
    return OEQ_OK;
}

// Mirror of oeq::UvuParams (uvu_kernels.cuh).
struct UvuParams {
    const void* X; const void* Y; const void* W; void* Z;
    const void* dZ; void* dX; void* dY; void* dW;
    const long long* rows; const long long* cols; const long long* perm;
    long long n_items, n_nodes;
    void* ws;
    int* status;
    int stages, flags, chunk;
    long long e_lo, e_hi;
    const long long* sum_cols; const long long* sum_perm; const void* sum_ws;
    long long sum_items, sum_e_lo, sum_e_hi;
    int sum_first, sum_chunk;
    const void* EX; const void* EY; const void* EW;
};

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

int launch_uvu(Kernel& k, const Problem& p, UvuParams& prm, cudaStream_t stream, int extra_flags = 0,
               long long max_ctas = 0, long long* ctas_out = nullptr, int clear_flags = 0) {
    const int e = p.elem();
    int flags = 0;
    if ((p.x_dim * e) % 16 == 0 && aligned16(prm.X)) flags |= 1;
    // (with several edges per item a bulk copy covers a run of rows: the run has to be a 16-byte multiple)
    const int epi = k.map.epi;
    if ((p.y_dim * e * epi) % 16 == 0 && aligned16(prm.Y)) flags |= 2;
    if (!p.shared && !p.unit && (p.w_numel * e * epi) % 16 == 0 && aligned16(prm.W)) flags |= 4;
    const void* zlike = prm.dZ ? prm.dZ : prm.Z;
    if ((p.z_dim * e) % 16 == 0 && aligned16(zlike)) flags |= 8;
    if (env_int("OEQ_B200_NO_BULK", 0)) flags = 0;
    flags &= ~clear_flags;
    {
        // short rows: 16-byte cp.async from all lanes instead of one bulk copy issued by one lane
        const int limit = env_int("OEQ_B200_VEC_COPY_BYTES", 0);
        const int row_bytes[4] = {p.x_dim * e, p.y_dim * e, p.w_numel * e, p.z_dim * e};
        for (int a = 0; a < 4; ++a)
            if ((flags & (1 << a)) && row_bytes[a] <= limit) flags = (flags & ~(1 << a)) | (256 << a);
    }
    prm.flags = flags | extra_flags;
    prm.stages = k.stages;
    long long want = (prm.n_items + k.map.ng - 1) / k.map.ng;
    long long grid = std::max<long long>(1, std::min<long long>((long long)k.sm_count * k.ctas_per_sm, want));
    if (max_ctas > 0) grid = std::min(grid, max_ctas);     // a caller with bounded scratch narrows the launch
    if (ctas_out) *ctas_out = grid;
    // chunks of consecutive edges are dealt round-robin to the groups: 128 edges unless that leaves a group fewer
    // than eight chunks (the last round then idles a large part of the machine)
    int chunk = env_int("OEQ_B200_CHUNK", 0);
    if (chunk <= 0) {
        chunk = 128;
        const long long groups = grid * k.map.ng;
        while (chunk > k.map.chunk_floor && prm.n_items / (groups * chunk) < 8) chunk /= 2;
    }
    prm.chunk = std::max(1, chunk);
    void* args[] = {&prm};
    OEQ_CUDA(cudaLaunchKernel((const void*)k.fn, dim3((unsigned)grid), dim3((unsigned)k.threads()), args,
                              (size_t)k.smem, stream));
    return OEQ_OK;
}

long long uvu_grid(const Kernel& k, long long n_items) {
    long long want = (n_items + k.map.ng - 1) / k.map.ng;
    return std::max<long long>(1, std::min<long long>((long long)k.sm_count * k.ctas_per_sm, want));
}

}  // namespace

// ====================================================================== C ABI

struct oeq_tp {
    Problem prob;
    Kernel fwd, bwd;
    Kernel fwd_tc;              // tensor-core forward ('uvw', shared FP32 weights), when the problem qualifies
    bool has_tc = false;
    Kernel bwd_dw_tc;           // tensor-core weight gradient of the same class of problems
    Kernel bwd_dxy_tc;          // tensor-core dX / dY of the same class of problems (when its tiles fit)
    bool has_bwd_tc = false, has_dxy_tc = false;
    Kernel dbl;                 // one-pass second derivatives ('uvu', per-row weights)
    bool has_dbl = false;
    TcBwdGeometry tc_bwd;
    void* d_packed_t = nullptr; // weights transposed, split and swizzled for the dX/dY kernel
    cudaKernel_t pack_t_fn = nullptr;
    TcGeometry tc;
    void* d_packed = nullptr;   // weights split and swizzled for the tensor cores (owned by the handle)
    cudaKernel_t pack_fn = nullptr;
    int* d_status = nullptr;
    cudaStream_t last_stream = nullptr;
};
struct oeq_conv {
    Problem prob;
    bool deterministic = false;
    Kernel fwd, bwd;
    Kernel fwd_tc;              // tensor-core forward pass, when the problem qualifies
    bool has_fwd_tc = false;
    Kernel bwd_recv;            // receiver-order backward pass (needs scratch in the deterministic variant)
    bool has_bwd_recv = false;
    cudaKernel_t sum_rows_fn = nullptr, clear_fn = nullptr;
    Kernel dbl_z, dbl_g;        // second derivatives in two launches; compiled at first use
    int dbl_state = 0;          // 0 not tried, 1 ready, -1 not available
    cudaKernel_t dbl_sum_fn = nullptr, dbl_clear_fn = nullptr;
    int last_bwd_launches = 0;  // kernel launches of the most recent oeq_conv_backward
    int* d_status = nullptr;
    cudaStream_t last_stream = nullptr;
};

extern "C" {

const char* oeq_version(void) { return "oeq_b200 0.1 (sm_100a)"; }
const char* oeq_last_error(void) { return g_error.c_str(); }

int oeq_set_kernel_dir(const char* path) {
    if (!path) return fail(OEQ_ERR_INVALID, "null path");
    g_kernel_dir = path;
    return OEQ_OK;
}
int oeq_set_cache_dir(const char* path) {
    if (!path) return fail(OEQ_ERR_INVALID, "null path");
    g_cache_dir = path;
    return OEQ_OK;
}

static int check_conv_problem(const Problem& p) {
    if (p.mode != OEQ_MODE_UVU) return fail(OEQ_ERR_UNSUPPORTED, "fused convolution supports 'uvu' problems only");
    if (p.shared) return fail(OEQ_ERR_UNSUPPORTED, "fused convolution needs per-edge weights (shared_weights=False)");
    // (shared_weights == 2, "every weight is 1", is a per-edge-weight problem without the array)
    for (const Irrep& r : p.in2)
        if (r.mul != 1) return fail(OEQ_ERR_UNSUPPORTED, "fused convolution needs multiplicity 1 for every irrep of the second input");
    return OEQ_OK;
}

int oeq_precompile(const oeq_problem_desc* desc, int kinds) {
    Problem p;
    int rc = ingest(desc, p);
    if (rc) return rc;
    if (p.mode == OEQ_MODE_UVW) {
        if (kinds & 6) return fail(OEQ_ERR_UNSUPPORTED, "fused convolution supports 'uvu' problems only");
        Kernel f, b, tc;
        if ((rc = build_tp(p, false, f)) || (rc = build_tp(p, true, b))) return rc;
        TcGeometry g;
        if (uvw_tc_geometry(p, g) && (rc = build_uvw_tc(p, tc))) return rc;
        TcBwdGeometry gb;
        Kernel dw, dxy;
        if (uvw_tc_bwd_geometry(p, gb)) {
            if ((rc = build_uvw_tc_bwd(p, K_UVW_TC_DW, dw))) return rc;
            if (gb.dxy_smem > 0 && (rc = build_uvw_tc_bwd(p, K_UVW_TC_DXY, dxy))) return rc;
        }
        return OEQ_OK;
    }
    auto one = [&](int kind) {
        Kernel k;
        return build_uvu(p, kind, k);
    };
    if (kinds & 1) {
        if ((rc = one(K_FWD_BATCH)) || (rc = one(K_BWD_BATCH))) return rc;
        if (double_backward_supported(p)) {
            Kernel k;
            rc = build_uvu_dbl(p, k);
            if (rc && rc != OEQ_ERR_UNSUPPORTED) return rc;
        }
    }
    if (kinds & 6) {
        if ((rc = check_conv_problem(p))) return rc;
    }
    UvuTcGeometry geo;
    const bool tc = (kinds & 6) && uvu_tc_geometry(p, geo);
    const bool recv = (kinds & 6) && recv_backward_supported(p);
    if (kinds & 2) {
        if ((rc = one(K_FWD_DET)) || (rc = one(K_BWD_DET))) return rc;
        Kernel k, kr;
        if (tc && (rc = build_uvu_tc(p, true, k))) return rc;
        if (recv && (rc = build_uvu_recv(p, true, kr))) return rc;
    }
    if (kinds & 4) {
        if ((rc = one(K_FWD_ATOMIC)) || (rc = one(K_BWD_ATOMIC))) return rc;
        Kernel k, kr;
        if (tc && (rc = build_uvu_tc(p, false, k))) return rc;
        if (recv && (rc = build_uvu_recv(p, false, kr))) return rc;
    }
    if ((kinds & 8) && (kinds & 6) && conv_double_backward_supported(p)) {
        for (int det = 0; det < 2; ++det) {
            if (!(kinds & (det ? 2 : 4))) continue;
            for (int grads = 0; grads < 2; ++grads) {
                Kernel k;
                rc = build_uvu_dblc(p, det != 0, grads != 0, k);
                if (rc && rc != OEQ_ERR_UNSUPPORTED) return rc;
            }
        }
    }
    return OEQ_OK;
}

// ---------------------------------------------------------------- batch TP

int oeq_tp_create(const oeq_problem_desc* desc, oeq_tp** out) {
    if (!out) return fail(OEQ_ERR_INVALID, "null output handle");
    *out = nullptr;
    oeq_tp* h = new oeq_tp();
    int rc = ingest(desc, h->prob);
    if (!rc) rc = build_tp(h->prob, false, h->fwd);
    if (!rc) rc = build_tp(h->prob, true, h->bwd);
    if (!rc && uvw_tc_geometry(h->prob, h->tc)) {
        rc = build_uvw_tc(h->prob, h->fwd_tc);
        h->has_tc = rc == OEQ_OK;
    }
    if (!rc && uvw_tc_bwd_geometry(h->prob, h->tc_bwd)) {
        rc = build_uvw_tc_bwd(h->prob, K_UVW_TC_DW, h->bwd_dw_tc);
        h->has_bwd_tc = rc == OEQ_OK;
        if (!rc && h->tc_bwd.dxy_smem > 0 && env_int("OEQ_B200_UVW_TC_DXY", 1)) {
            rc = build_uvw_tc_bwd(h->prob, K_UVW_TC_DXY, h->bwd_dxy_tc);
            h->has_dxy_tc = rc == OEQ_OK;
        }
    }
    if (!rc && double_backward_supported(h->prob)) {
        const int rc2 = build_uvu_dbl(h->prob, h->dbl);
        if (rc2 == OEQ_OK) h->has_dbl = true;
        else if (rc2 != OEQ_ERR_UNSUPPORTED) rc = rc2;
    }
    if (rc) {
        delete h;
        return rc;
    }
    *out = h;
    return OEQ_OK;
}

int oeq_tp_destroy(oeq_tp* h) {
    if (!h) return OEQ_OK;
    if (h->d_status) cudaFree(h->d_status);
    if (h->d_packed) cudaFree(h->d_packed);
    if (h->d_packed_t) cudaFree(h->d_packed_t);
    for (Kernel* k : {&h->fwd, &h->bwd, &h->fwd_tc, &h->bwd_dw_tc, &h->bwd_dxy_tc, &h->dbl})
        if (k->lib) cudaLibraryUnload(k->lib);
    delete h;
    return OEQ_OK;
}

int64_t oeq_tp_weight_numel(const oeq_tp* h) { return h ? h->prob.w_numel : -1; }

static int ensure_status(int** d_status) {
    if (*d_status) return OEQ_OK;
    OEQ_CUDA(cudaMalloc(d_status, sizeof(int)));
    OEQ_CUDA(cudaMemset(*d_status, 0, sizeof(int)));
    return OEQ_OK;
}

int oeq_tp_forward(oeq_tp* h, int64_t batch, const void* X, const void* Y, const void* W, void* Z, void* stream) {
    if (!h) return fail(OEQ_ERR_INVALID, "null handle");
    if (batch < 0) return fail(OEQ_ERR_INVALID, "negative batch");
    if (batch == 0) return OEQ_OK;
    if (!X || !Y || !W || !Z) return fail(OEQ_ERR_INVALID, "null buffer");
    int rc = ensure_status(&h->d_status);
    if (rc) return rc;
    h->last_stream = (cudaStream_t)stream;
    if (h->has_tc) {
        Kernel& k = h->fwd_tc;
        cudaStream_t st = (cudaStream_t)stream;
        if (!k.loaded) {
            OEQ_CUDA(cudaLibraryLoadData(&k.lib, k.code.cubin.data(), nullptr, nullptr, 0, nullptr, nullptr, 0));
            OEQ_CUDA(cudaLibraryGetKernel(&k.fn, k.lib, "oeq_uvw_tc_kernel"));
            OEQ_CUDA(cudaLibraryGetKernel(&h->pack_fn, k.lib, "oeq_uvw_pack_weights"));
            int dev = 0;
            OEQ_CUDA(cudaGetDevice(&dev));
            OEQ_CUDA(cudaDeviceGetAttribute(&k.sm_count, cudaDevAttrMultiProcessorCount, dev));
            k.smem = h->tc.smem;
            OEQ_CUDA(cudaFuncSetAttribute((const void*)k.fn, cudaFuncAttributeMaxDynamicSharedMemorySize, k.smem));
            cudaFuncAttributes attr;
            if (cudaFuncGetAttributes(&attr, (const void*)k.fn) == cudaSuccess) k.regs = attr.numRegs;
            else (void)cudaGetLastError();
            OEQ_CUDA(cudaMalloc(&h->d_packed, h->tc.packed_bytes));
            k.loaded = true;
        }
        {
            void* packed = h->d_packed;
            void* args[] = {(void*)&W, &packed};
            OEQ_CUDA(cudaLaunchKernel((const void*)h->pack_fn, dim3(64), dim3(256), args, 0, st));
        }
        struct { const void* X; const void* Y; const void* Wp; void* Z; long long batch; int* status; unsigned long long* prof; }
            tp{X, Y, h->d_packed, Z, batch, h->d_status, nullptr};
        void* args[] = {&tp};
        const long long grid = std::max<long long>(1, std::min<long long>(k.sm_count, (batch + 23) / 24));
#ifdef OEQ_DEV_PROFILE
        if (env_int("OEQ_B200_TC_PROFILE", 0)) {
            // cycle accounting of the roles of CTA 0 (development aid): synchronous, prints to stderr
            OEQ_CUDA(cudaMalloc(&tp.prof, 32 * 8));
            OEQ_CUDA(cudaMemsetAsync(tp.prof, 0, 32 * 8, st));
            OEQ_CUDA(cudaLaunchKernel((const void*)k.fn, dim3((unsigned)grid), dim3(21 * 32), args, (size_t)k.smem, st));
            unsigned long long hb[32];
            OEQ_CUDA(cudaMemcpyAsync(hb, tp.prof, sizeof hb, cudaMemcpyDeviceToHost, st));
            OEQ_CUDA(cudaStreamSynchronize(st));
            cudaFree(tp.prof);
            fprintf(stderr, "[oeq_b200 uvw tc profile] producer: stages %llu wait %llu fill %llu | mma: wait %llu issue %llu | "
                            "epilogue: tiles %llu wait %llu drain %llu\n", hb[2], hb[0], hb[1], hb[8], hb[9], hb[18], hb[16], hb[17]);
            return OEQ_OK;
        }
#endif
        OEQ_CUDA(cudaLaunchKernel((const void*)k.fn, dim3((unsigned)grid), dim3(21 * 32), args, (size_t)k.smem, st));
        return OEQ_OK;
    }
    if (h->prob.mode == OEQ_MODE_UVW) {
        if ((rc = load_uvw(h->fwd, h->prob, false))) return rc;
        UvwParams up{};
        up.X = X; up.Y = Y; up.W = W; up.Z = Z; up.batch = batch; up.status = h->d_status;
        void* args[] = {&up};
        OEQ_CUDA(cudaLaunchKernel((const void*)h->fwd.fn, dim3((unsigned)uvw_grid(h->fwd, batch)),
                                  dim3((unsigned)h->fwd.uvw.threads), args, (size_t)h->fwd.smem, (cudaStream_t)stream));
        return OEQ_OK;
    }
    if ((rc = load_kernel(h->fwd, "oeq_uvu_kernel", false))) return rc;
    UvuParams prm{};
    prm.X = X; prm.Y = Y; prm.W = W; prm.Z = Z;
    prm.n_items = batch; prm.n_nodes = batch; prm.status = h->d_status;
    return launch_uvu(h->fwd, h->prob, prm, (cudaStream_t)stream);
}

size_t oeq_tp_workspace_bytes(const oeq_tp* h, int64_t batch) {
    if (!h || !h->prob.shared || batch <= 0) return 0;
    // one partial weight gradient per group (uvu) or per CTA (uvw) of the backward launch; sized for the
    // largest grid the launch can use on any device (256 SMs)
    long long groups;
    if (h->prob.mode == OEQ_MODE_UVW) {
        const long long tiles = (batch + h->bwd.uvw.tile_r - 1) / h->bwd.uvw.tile_r;
        groups = std::max<long long>(std::min<long long>(tiles, 256ll * 2), h->has_bwd_tc ? 256ll : 0ll);
    } else {
        groups = 256ll * 4 * h->bwd.map.ng;
    }
    return (size_t)groups * h->prob.w_numel * h->prob.elem();
}

int oeq_tp_backward(oeq_tp* h, int64_t batch, const void* X, const void* Y, const void* W, const void* dZ, void* dX,
                    void* dY, void* dW, void* workspace, size_t workspace_bytes, void* stream) {
    if (!h) return fail(OEQ_ERR_INVALID, "null handle");
    if (batch < 0) return fail(OEQ_ERR_INVALID, "negative batch");
    cudaStream_t st = (cudaStream_t)stream;
    const Problem& p = h->prob;
    if (batch == 0) {
        if (p.shared && dW) OEQ_CUDA(cudaMemsetAsync(dW, 0, (size_t)p.w_numel * p.elem(), st));
        return OEQ_OK;
    }
    if (!X || !Y || !W || !dZ || !dX || !dY || !dW) return fail(OEQ_ERR_INVALID, "null buffer");
    int rc = ensure_status(&h->d_status);
    if (rc) return rc;
    if (p.mode == OEQ_MODE_UVW) {
        if ((rc = load_uvw(h->bwd, p, true))) return rc;
        long long ctas = uvw_grid(h->bwd, batch);
        if (p.shared) {
            const size_t need = (size_t)ctas * p.w_numel * p.elem();
            if (!workspace || workspace_bytes < need)
                return fail(OEQ_ERR_INVALID, "workspace too small for the shared-weight gradient (see oeq_tp_workspace_bytes)");
        }
        UvwParams up{};
        up.X = X; up.Y = Y; up.W = W; up.dZ = dZ; up.dX = dX; up.dY = dY; up.dW = dW; up.ws = workspace;
        up.batch = batch; up.status = h->d_status;
        h->last_stream = st;
        if (h->has_bwd_tc) {
            // weight gradient on the tensor cores (per-CTA partial sums in the workspace, then the fixed-order
            // reduction); the FMA kernel computes dX and dY only
            Kernel& k = h->bwd_dw_tc;
            if (!k.loaded) {
                OEQ_CUDA(cudaLibraryLoadData(&k.lib, k.code.cubin.data(), nullptr, nullptr, 0, nullptr, nullptr, 0));
                OEQ_CUDA(cudaLibraryGetKernel(&k.fn, k.lib, "oeq_uvw_tc_dw_kernel"));
                OEQ_CUDA(cudaLibraryGetKernel(&k.reduce_fn, k.lib, "oeq_reduce_partials"));
                int dev = 0;
                OEQ_CUDA(cudaGetDevice(&dev));
                OEQ_CUDA(cudaDeviceGetAttribute(&k.sm_count, cudaDevAttrMultiProcessorCount, dev));
                k.smem = h->tc_bwd.dw_smem;
                OEQ_CUDA(cudaFuncSetAttribute((const void*)k.fn, cudaFuncAttributeMaxDynamicSharedMemorySize, k.smem));
                k.loaded = true;
            }
            long long dw_ctas = std::max<long long>(1, std::min<long long>(k.sm_count, (batch + 31) / 32));
            if ((size_t)dw_ctas * p.w_numel * p.elem() > workspace_bytes)
                return fail(OEQ_ERR_INVALID, "workspace too small for the shared-weight gradient (see oeq_tp_workspace_bytes)");
            struct { const void* X; const void* Y; const void* Wt; const void* dZ; void* dX; void* dY; void* ws; long long batch;
                     int* status; unsigned long long* prof; } tp{X, Y, nullptr, dZ, dX, dY, workspace, batch, h->d_status, nullptr};
            void* targs[] = {&tp};
            OEQ_CUDA(cudaLaunchKernel((const void*)k.fn, dim3((unsigned)dw_ctas), dim3(21 * 32), targs, (size_t)k.smem, st));
            int n = p.w_numel;
            const void* ws = workspace;
            void* rargs[] = {&ws, &dW, &n, &dw_ctas};
            OEQ_CUDA(cudaLaunchKernel((const void*)k.reduce_fn, dim3((n + 127) / 128), dim3(128), rargs, 0, st));
            up.skip_dw = 1;
            up.ws = nullptr;
            if (h->has_dxy_tc) {
                // dX and dY on the tensor cores too: the FMA kernel is not launched at all
                Kernel& kx = h->bwd_dxy_tc;
                if (!kx.loaded) {
                    OEQ_CUDA(cudaLibraryLoadData(&kx.lib, kx.code.cubin.data(), nullptr, nullptr, 0, nullptr, nullptr, 0));
                    OEQ_CUDA(cudaLibraryGetKernel(&kx.fn, kx.lib, "oeq_uvw_tc_dxy_kernel"));
                    OEQ_CUDA(cudaLibraryGetKernel(&h->pack_t_fn, kx.lib, "oeq_uvw_pack_weights_t"));
                    kx.sm_count = k.sm_count;
                    kx.smem = h->tc_bwd.dxy_smem;
                    OEQ_CUDA(cudaFuncSetAttribute((const void*)kx.fn, cudaFuncAttributeMaxDynamicSharedMemorySize, kx.smem));
                    OEQ_CUDA(cudaMalloc(&h->d_packed_t, h->tc_bwd.wt_bytes));
                    kx.loaded = true;
                }
                void* packed = h->d_packed_t;
                void* pargs[] = {(void*)&W, &packed};
                OEQ_CUDA(cudaLaunchKernel((const void*)h->pack_t_fn, dim3(64), dim3(256), pargs, 0, st));
                OEQ_CUDA(cudaMemsetAsync(dX, 0, (size_t)batch * p.x_dim * p.elem(), st));
                OEQ_CUDA(cudaMemsetAsync(dY, 0, (size_t)batch * p.y_dim * p.elem(), st));
                tp.Wt = h->d_packed_t;
                const long long ctas_x = std::max<long long>(1, std::min<long long>(kx.sm_count, (batch + 23) / 24));
#ifdef OEQ_DEV_PROFILE
                if (env_int("OEQ_B200_TC_PROFILE", 0)) {
                    // cycle accounting of the roles of CTA 0 (development aid): synchronous, prints to stderr
                    OEQ_CUDA(cudaMalloc(&tp.prof, 32 * 8));
                    OEQ_CUDA(cudaMemsetAsync(tp.prof, 0, 32 * 8, st));
                    OEQ_CUDA(cudaLaunchKernel((const void*)kx.fn, dim3((unsigned)ctas_x), dim3(16 * 32), targs, (size_t)kx.smem, st));
                    unsigned long long hb[32];
                    OEQ_CUDA(cudaMemcpyAsync(hb, tp.prof, sizeof hb, cudaMemcpyDeviceToHost, st));
                    OEQ_CUDA(cudaStreamSynchronize(st));
                    cudaFree(tp.prof);
                    fprintf(stderr, "[oeq_b200 uvw dxy profile] producer: stages %llu wait %llu fill %llu | mma: wait-acc %llu wait-full %llu "
                                    "issue %llu | epilogue: wait %llu drain %llu rows %llu sync %llu | per row: n %llu compute %llu dy %llu\n", hb[2], hb[0], hb[1], hb[8], hb[9],
                            hb[10], hb[16], hb[17], hb[18], hb[19], hb[26], hb[24], hb[25]);
                    return OEQ_OK;
                }
#endif
                OEQ_CUDA(cudaLaunchKernel((const void*)kx.fn, dim3((unsigned)ctas_x), dim3(16 * 32), targs, (size_t)kx.smem, st));
                return OEQ_OK;
            }
        }
        void* args[] = {&up};
        OEQ_CUDA(cudaLaunchKernel((const void*)h->bwd.fn, dim3((unsigned)ctas), dim3((unsigned)h->bwd.uvw.threads), args,
                                  (size_t)h->bwd.smem, st));
        if (p.shared && !h->has_bwd_tc) {
            int n = p.w_numel;
            const void* ws = workspace;
            void* rargs[] = {&ws, &dW, &n, &ctas};
            OEQ_CUDA(cudaLaunchKernel((const void*)h->bwd.reduce_fn, dim3((n + 127) / 128), dim3(128), rargs, 0, st));
        }
        return OEQ_OK;
    }
    if ((rc = load_kernel(h->bwd, "oeq_uvu_kernel", true))) return rc;
    UvuParams prm{};
    prm.X = X; prm.Y = Y; prm.W = W; prm.dZ = dZ; prm.dX = dX; prm.dY = dY; prm.dW = dW;
    prm.n_items = batch; prm.n_nodes = batch; prm.status = h->d_status;
    long long groups = 0;
    if (p.shared) {
        groups = uvu_grid(h->bwd, batch) * h->bwd.map.ng;
        const size_t need = (size_t)groups * p.w_numel * p.elem();
        if (!workspace || workspace_bytes < need)
            return fail(OEQ_ERR_INVALID, "workspace too small for the shared-weight gradient (see oeq_tp_workspace_bytes)");
        prm.ws = workspace;
    }
    h->last_stream = st;
    rc = launch_uvu(h->bwd, p, prm, st);
    if (rc) return rc;
    if (p.shared) {
        int n = p.w_numel;
        const void* ws = workspace;
        void* args[] = {&ws, &dW, &n, &groups};
        OEQ_CUDA(cudaLaunchKernel((const void*)h->bwd.reduce_fn, dim3((n + 127) / 128), dim3(128), args, 0, st));
    }
    return OEQ_OK;
}

int oeq_tp_has_double_backward(const oeq_tp* h) { return h && h->has_dbl ? 1 : 0; }

int oeq_tp_double_backward(oeq_tp* h, int64_t batch, const void* X, const void* Y, const void* W, const void* dZ,
                           const void* EX, const void* EY, const void* EW, void* GX, void* GY, void* GW, void* GdZ,
                           void* stream) {
    if (!h) return fail(OEQ_ERR_INVALID, "null handle");
    if (!h->has_dbl) return fail(OEQ_ERR_UNSUPPORTED, "no one-pass second-derivative kernel for this problem: compose it from "
                                                      "oeq_tp_forward and oeq_tp_backward");
    if (batch < 0) return fail(OEQ_ERR_INVALID, "negative batch");
    if (batch == 0) return OEQ_OK;
    if (!X || !Y || !W || !dZ || !EX || !EY || !EW || !GX || !GY || !GW || !GdZ) return fail(OEQ_ERR_INVALID, "null buffer");
    int rc = ensure_status(&h->d_status);
    if (!rc) rc = load_kernel(h->dbl, "oeq_uvu_kernel", false);
    if (rc) return rc;
    const Problem& p = h->prob;
    const int e = p.elem();
    UvuParams prm{};
    prm.X = X; prm.Y = Y; prm.W = W; prm.dZ = dZ; prm.EX = EX; prm.EY = EY; prm.EW = EW;
    prm.dX = GX; prm.dY = GY; prm.dW = GW; prm.Z = GdZ;
    prm.n_items = batch; prm.n_nodes = batch; prm.status = h->d_status;
    h->last_stream = (cudaStream_t)stream;
    // launch_uvu derives the bulk-copy bits from X, Y, W, dZ; a cotangent that breaks the 16-byte rule clears
    // the bit of its pair
    int clear = 0;
    if (!aligned16(EX)) clear |= 1;
    if (!aligned16(EY)) clear |= 2;
    if (!aligned16(EW)) clear |= 4;
    (void)e;
    return launch_uvu(h->dbl, p, prm, (cudaStream_t)stream, 0, 0, nullptr, clear);
}

static int check_status(int* d_status, cudaStream_t st) {
    if (!d_status) return OEQ_OK;
    int v = 0;
    OEQ_CUDA(cudaStreamSynchronize(st));
    OEQ_CUDA(cudaMemcpy(&v, d_status, sizeof v, cudaMemcpyDeviceToHost));
    if (v != 0) {
        cudaMemset(d_status, 0, sizeof v);
        return fail(OEQ_ERR_DEVICE_WAIT, "a kernel abandoned a bounded wait (code " + std::to_string(v) + ")");
    }
    return OEQ_OK;
}
int oeq_tp_check(oeq_tp* h) { return h ? check_status(h->d_status, h->last_stream) : fail(OEQ_ERR_INVALID, "null handle"); }

static int launch_info(const Kernel& k, int* threads, int* ng, int* ps, int* stages, int* smem, int* regs) {
    if (threads) *threads = k.is_uvw ? k.uvw.threads : k.threads();
    if (ng) *ng = k.map.ng;
    if (ps) *ps = k.map.ps;
    if (stages) *stages = k.stages;
    if (smem) *smem = k.smem;
    if (regs) *regs = k.regs;
    return OEQ_OK;
}
int oeq_tp_launch_info(const oeq_tp* h, int which, int* threads, int* ng, int* ps, int* stages, int* smem, int* regs) {
    if (!h) return fail(OEQ_ERR_INVALID, "null handle");
    if (!which && h->has_tc) {
        if (threads) *threads = 21 * 32;
        if (ng) *ng = 1;
        if (ps) *ps = 1;
        if (stages) *stages = 2;
        if (smem) *smem = h->fwd_tc.smem;
        if (regs) *regs = h->fwd_tc.regs;
        return OEQ_OK;
    }
    return launch_info(which ? h->bwd : h->fwd, threads, ng, ps, stages, smem, regs);
}

// ---------------------------------------------------------------- backward pass that allocates nothing

// Scratch for oeq_tp_backward_noalloc: lives in the library image, so every GPU that loads the
// library holds these bytes until the process exits.
constexpr size_t NOALLOC_SCRATCH_BYTES = 8u << 20;
static __device__ __align__(256) unsigned char g_noalloc_scratch[NOALLOC_SCRATCH_BYTES];
// In host code the array's name only stands for the symbol; the device address is looked up
// once per device (with that device current) and remembered here.
static void* g_noalloc_scratch_addr[64] = {nullptr};
static std::mutex g_noalloc_mutex;

static int noalloc_scratch(void** out) {
    int dev = 0;
    OEQ_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(OEQ_ERR_INVALID, "device ordinal out of range");
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);     // two host threads may make a device's first call at once
    if (!g_noalloc_scratch_addr[dev]) {
        void* ptr = nullptr;
        OEQ_CUDA(cudaGetSymbolAddress(&ptr, g_noalloc_scratch));
        g_noalloc_scratch_addr[dev] = ptr;
    }
    *out = g_noalloc_scratch_addr[dev];
    return OEQ_OK;
}

int oeq_tp_backward_noalloc(oeq_tp* h, int64_t batch, const void* X, const void* Y, const void* W, const void* dZ,
                            void* dX, void* dY, void* dW, void* stream) {
    if (!h) return fail(OEQ_ERR_INVALID, "null handle");
    const Problem& p = h->prob;
    if (!p.shared)
        return fail(OEQ_ERR_INVALID, "per-row weights need no scratch: call oeq_tp_backward with a null workspace");
    if (batch <= 0) return fail(OEQ_ERR_INVALID, "batch must be positive");
    if (!X || !Y || !W || !dZ || !dX || !dY || !dW) return fail(OEQ_ERR_INVALID, "null buffer");
    const size_t slice = (size_t)p.w_numel * p.elem();
    if (slice == 0 || slice > NOALLOC_SCRATCH_BYTES)
        return fail(OEQ_ERR_UNSUPPORTED, "weight tensor of " + std::to_string(slice) + " bytes exceeds the built-in scratch of " +
                                             std::to_string(NOALLOC_SCRATCH_BYTES) + " bytes; use oeq_tp_backward with caller scratch");
    const long long max_slices = (long long)(NOALLOC_SCRATCH_BYTES / slice);
    cudaStream_t st = (cudaStream_t)stream;
    void* scratch = nullptr;
    int rc = noalloc_scratch(&scratch);
    if (rc) return rc;
    h->last_stream = st;       // oeq_tp_check synchronises the stream of the most recent launch
    if (p.mode == OEQ_MODE_UVW) {
        // always the FMA kernel: the tensor-core kernels want packed weight copies that only cudaMalloc gives
        if ((rc = load_uvw(h->bwd, p, true))) return rc;
        long long ctas = std::min(uvw_grid(h->bwd, batch), max_slices);
        UvwParams up{};
        up.X = X; up.Y = Y; up.W = W; up.dZ = dZ; up.dX = dX; up.dY = dY; up.dW = dW; up.ws = scratch;
        up.batch = batch; up.status = h->d_status;
        void* args[] = {&up};
        OEQ_CUDA(cudaLaunchKernel((const void*)h->bwd.fn, dim3((unsigned)ctas), dim3((unsigned)h->bwd.uvw.threads), args,
                                  (size_t)h->bwd.smem, st));
        int n = p.w_numel;
        const void* ws = scratch;
        void* rargs[] = {&ws, &dW, &n, &ctas};
        OEQ_CUDA(cudaLaunchKernel((const void*)h->bwd.reduce_fn, dim3((n + 127) / 128), dim3(128), rargs, 0, st));
        return OEQ_OK;
    }
    if ((rc = load_kernel(h->bwd, "oeq_uvu_kernel", true))) return rc;
    Kernel& k = h->bwd;
    const long long max_ctas = max_slices / k.map.ng;
    if (max_ctas < 1)
        return fail(OEQ_ERR_UNSUPPORTED, "one CTA's partial gradients exceed the built-in scratch; use oeq_tp_backward");
    UvuParams prm{};
    prm.X = X; prm.Y = Y; prm.W = W; prm.dZ = dZ; prm.dX = dX; prm.dY = dY; prm.dW = dW;
    prm.n_items = batch; prm.n_nodes = batch; prm.status = h->d_status; prm.ws = scratch;
    long long grid = 0;
    if ((rc = launch_uvu(k, p, prm, st, 0, max_ctas, &grid))) return rc;
    long long groups = grid * k.map.ng;
    int n = p.w_numel;
    const void* ws = scratch;
    void* rargs[] = {&ws, &dW, &n, &groups};
    OEQ_CUDA(cudaLaunchKernel((const void*)k.reduce_fn, dim3((n + 127) / 128), dim3(128), rargs, 0, st));
    return OEQ_OK;
}

// ---------------------------------------------------------------- fused convolution

int oeq_conv_create(const oeq_problem_desc* desc, int deterministic, oeq_conv** out) {
    if (!out) return fail(OEQ_ERR_INVALID, "null output handle");
    *out = nullptr;
    oeq_conv* h = new oeq_conv();
    h->deterministic = deterministic != 0;
    int rc = ingest(desc, h->prob);
    if (!rc) rc = check_conv_problem(h->prob);
    if (!rc) rc = build_uvu(h->prob, deterministic ? K_FWD_DET : K_FWD_ATOMIC, h->fwd);
    if (!rc) rc = build_uvu(h->prob, deterministic ? K_BWD_DET : K_BWD_ATOMIC, h->bwd);
    UvuTcGeometry geo;
    if (!rc && uvu_tc_geometry(h->prob, geo)) {
        rc = build_uvu_tc(h->prob, h->deterministic, h->fwd_tc);
        h->has_fwd_tc = !rc;
    }
    if (!rc && recv_backward_supported(h->prob)) {
        rc = build_uvu_recv(h->prob, h->deterministic, h->bwd_recv);
        h->has_bwd_recv = !rc;
    }
    if (rc) {
        delete h;
        return rc;
    }
    *out = h;
    return OEQ_OK;
}

int oeq_conv_destroy(oeq_conv* h) {
    if (!h) return OEQ_OK;
    if (h->d_status) cudaFree(h->d_status);
    if (h->fwd.lib) cudaLibraryUnload(h->fwd.lib);
    if (h->bwd.lib) cudaLibraryUnload(h->bwd.lib);
    if (h->fwd_tc.lib) cudaLibraryUnload(h->fwd_tc.lib);
    if (h->bwd_recv.lib) cudaLibraryUnload(h->bwd_recv.lib);
    if (h->dbl_z.lib) cudaLibraryUnload(h->dbl_z.lib);
    if (h->dbl_g.lib) cudaLibraryUnload(h->dbl_g.lib);
    delete h;
    return OEQ_OK;
}

// Scratch row of one edge in the deterministic receiver-order backward pass.
static size_t recv_row_bytes(const Problem& p) { return (size_t)pad16(p.x_dim * p.elem()); }
// Below this many scratch rows (when the edges do not all fit) the sender-order kernel is used instead.
static long long recv_min_block_edges() { return std::max(1, env_int("OEQ_B200_BWD_MIN_BLOCK", 1 << 16)); }

size_t oeq_conv_workspace_bytes(const oeq_conv* h, int64_t nodes, int64_t edges) {
    (void)nodes;
    // Forward: none (the segmented reduction is node-aligned: no scratch, no fix-up pass).  Deterministic
    // backward: one dX row per edge, capped (the pass then runs over blocks of edges); optional -- without
    // it the sender-order kernel runs.
    if (!h || !h->deterministic || !h->has_bwd_recv || edges <= 0) return 0;
    const size_t cap = (size_t)std::max(1, env_int("OEQ_B200_BWD_SCRATCH_MB", 8192)) << 20;
    return std::min((size_t)edges * recv_row_bytes(h->prob), cap);
}

int oeq_conv_forward(oeq_conv* h, int64_t nodes, int64_t edges, const void* X, const void* Y, const void* W,
                     const int64_t* rows, const int64_t* cols, void* Z, void* workspace, size_t workspace_bytes,
                     void* stream) {
    (void)workspace; (void)workspace_bytes;
    if (!h) return fail(OEQ_ERR_INVALID, "null handle");
    if (nodes < 0 || edges < 0) return fail(OEQ_ERR_INVALID, "negative size");
    cudaStream_t st = (cudaStream_t)stream;
    const Problem& p = h->prob;
    if (nodes == 0) return OEQ_OK;
    if (!Z) return fail(OEQ_ERR_INVALID, "null buffer");
    if (edges == 0 || !h->deterministic)
        OEQ_CUDA(cudaMemsetAsync(Z, 0, (size_t)nodes * p.z_dim * p.elem(), st));
    if (edges == 0) return OEQ_OK;
    if (!X || !Y || (!W && !p.unit) || !rows || !cols) return fail(OEQ_ERR_INVALID, "null buffer");
    // the tensor-core kernel stages rows with bulk copies only: it needs 16-byte aligned X and W
    const bool tc = h->has_fwd_tc && aligned16(X) && aligned16(W) && !env_int("OEQ_B200_NO_BULK", 0);
    int rc = ensure_status(&h->d_status);
    if (!rc) rc = tc ? load_kernel(h->fwd_tc, "oeq_uvu_tc_kernel", false) : load_kernel(h->fwd, "oeq_uvu_kernel", false);
    if (rc) return rc;
    UvuParams prm{};
    prm.X = X; prm.Y = Y; prm.W = W; prm.Z = Z;
    prm.rows = (const long long*)rows; prm.cols = (const long long*)cols;
    prm.n_items = edges; prm.n_nodes = nodes; prm.status = h->d_status;
    h->last_stream = st;
#ifdef OEQ_DEV_PROFILE
    if (tc && env_int("OEQ_B200_TC_PROFILE", 0)) {
        // cycle accounting of the roles of CTA 0 (development aid): synchronous, prints to stderr
        unsigned long long* d = nullptr;
        OEQ_CUDA(cudaMalloc(&d, 64 * 8));
        OEQ_CUDA(cudaMemsetAsync(d, 0, 64 * 8, st));
        prm.ws = d;
        rc = launch_uvu(h->fwd_tc, p, prm, st);
        unsigned long long hbuf[64];
        OEQ_CUDA(cudaMemcpyAsync(hbuf, d, sizeof hbuf, cudaMemcpyDeviceToHost, st));
        OEQ_CUDA(cudaStreamSynchronize(st));
        cudaFree(d);
        const char* names[] = {"consumer0", "consumer1", "mma", "-", "stager"};
        for (int r = 0; r < 5; ++r)
            fprintf(stderr, "[oeq_b200 tc profile] %-9s total %llu  s1 %llu  s2 %llu  s3 %llu  s4 %llu  s5 %llu  s6 %llu  s7 %llu\n",
                    names[r], hbuf[8 * r], hbuf[8 * r + 1], hbuf[8 * r + 2], hbuf[8 * r + 3], hbuf[8 * r + 4], hbuf[8 * r + 5],
                    hbuf[8 * r + 6], hbuf[8 * r + 7]);
        return rc;
    }
#endif
    return launch_uvu(tc ? h->fwd_tc : h->fwd, p, prm, st);
}

int oeq_conv_backward(oeq_conv* h, int64_t nodes, int64_t edges, const void* X, const void* Y, const void* W,
                      const void* dZ, const int64_t* rows, const int64_t* cols, const int64_t* perm, void* dX,
                      void* dY, void* dW, void* workspace, size_t workspace_bytes, void* stream) {
    if (!h) return fail(OEQ_ERR_INVALID, "null handle");
    if (nodes < 0 || edges < 0) return fail(OEQ_ERR_INVALID, "negative size");
    cudaStream_t st = (cudaStream_t)stream;
    const Problem& p = h->prob;
    if (nodes == 0) return OEQ_OK;
    if (!dX) return fail(OEQ_ERR_INVALID, "null buffer");
    if (edges == 0 || !h->deterministic)
        OEQ_CUDA(cudaMemsetAsync(dX, 0, (size_t)nodes * p.x_dim * p.elem(), st));
    if (edges == 0) return OEQ_OK;
    if (!X || !Y || !dZ || !rows || !cols || !dY || ((!W || !dW) && !p.unit))
        return fail(OEQ_ERR_INVALID, "null buffer");
    if (h->deterministic && !perm)
        return fail(OEQ_ERR_INVALID, "deterministic backward needs the sender-order permutation");
    int rc = ensure_status(&h->d_status);
    if (rc) return rc;
    h->last_stream = st;
    const int e = p.elem();
    // receiver-order pass: atomic variant always (dX was cleared above); deterministic variant when the
    // caller's scratch holds the rows of a useful block of edges
    const size_t row = recv_row_bytes(p);
    long long block_edges = 0;
    if (h->has_bwd_recv) {
        if (!h->deterministic) block_edges = edges;
        else if (workspace && aligned16(workspace)) {
            block_edges = (long long)std::min<size_t>(workspace_bytes / row, (size_t)edges);
            if (block_edges < edges && block_edges < recv_min_block_edges()) block_edges = 0;
        }
    }
    if (block_edges > 0) {
        Kernel& k = h->bwd_recv;
        if (!k.loaded) {
            if ((rc = load_kernel(k, "oeq_uvu_kernel", false))) return rc;
            if (h->deterministic) {
                OEQ_CUDA(cudaLibraryGetKernel(&h->sum_rows_fn, k.lib, "oeq_sum_sender_rows"));
                OEQ_CUDA(cudaLibraryGetKernel(&h->clear_fn, k.lib, "oeq_clear"));
            }
        }
        const char* Yb = (const char*)Y; const char* Wb = (const char*)W;
        char* dYb = (char*)dY; char* dWb = (char*)dW;
        h->last_bwd_launches = 0;
        const int dx_bulk = ((p.x_dim * e) % 16 == 0 && aligned16(dX)) ? 32 : 0;
        const int sum_chunk = std::max(1, env_int("OEQ_B200_SUM_CHUNK", 64));
        auto pass1 = [&](long long e0, long long n, void* scratch, UvuParams& prm) {
            prm.X = X; prm.dZ = dZ; prm.dX = dX;
            prm.Y = Yb + (size_t)e0 * p.y_dim * e; prm.W = Wb + (size_t)e0 * p.w_numel * e;
            prm.dY = dYb + (size_t)e0 * p.y_dim * e; prm.dW = dWb + (size_t)e0 * p.w_numel * e;
            prm.rows = (const long long*)rows + e0; prm.cols = (const long long*)cols + e0;
            prm.n_items = n; prm.n_nodes = nodes; prm.status = h->d_status;
            prm.ws = scratch;
        };
        if (!h->deterministic) {
            UvuParams prm{};
            pass1(0, edges, nullptr, prm);
            if ((rc = launch_uvu(k, p, prm, st, dx_bulk))) return rc;
            h->last_bwd_launches = 1;
            return OEQ_OK;
        }
        // rows of nodes that send nothing are never written by the row sum (cleared by a kernel: a memset call
        // may land on a copy engine behind the caller's host transfers)
        {
            unsigned long long words = (unsigned long long)nodes * p.x_dim * e / 4;
            void* ptr = dX;
            void* args[] = {&ptr, &words};
            const unsigned grid = (unsigned)std::max<unsigned long long>(1, std::min<unsigned long long>((unsigned long long)k.sm_count * 8, (words / 4 + 255) / 256));
            OEQ_CUDA(cudaLaunchKernel((const void*)h->clear_fn, dim3(grid), dim3(256), args, 0, st));
            ++h->last_bwd_launches;
        }
        auto sum_launch = [&](long long e0, long long n, void* scratch, bool first) -> int {
            UvuParams sp{};
            sp.dX = dX; sp.ws = scratch;
            sp.rows = (const long long*)rows; sp.cols = (const long long*)cols; sp.perm = (const long long*)perm;
            sp.n_items = edges; sp.n_nodes = nodes; sp.status = h->d_status;
            sp.flags = first ? 64 : 0;
            sp.chunk = sum_chunk;
            sp.e_lo = e0; sp.e_hi = e0 + n;
            const long long chunks = (edges + sp.chunk - 1) / sp.chunk;
            const long long grid = std::max<long long>(1, std::min<long long>((long long)k.sm_count * 6, (chunks + 7) / 8));
            void* args[] = {&sp};
            OEQ_CUDA(cudaLaunchKernel((const void*)h->sum_rows_fn, dim3((unsigned)grid), dim3(256), args, 0, st));
            ++h->last_bwd_launches;
            return OEQ_OK;
        };
        // With helper warps the scratch is used as two halves: launch b writes the rows of block b into half
        // b % 2 while its helper warps sum block b - 1 from the other half; the last block is summed by a
        // launch of its own.  Blocks are kept above a minimum size, and a list that fits one half is still cut
        // into a few blocks so that most of the summing hides behind the receiver-order launches.
        // Pipelining pays when a block's receiver-order launch runs for a millisecond or more; the scratch
        // bytes of a block are a fair proxy for that (wide rows mean much arithmetic per edge).
        const size_t min_block_bytes = (size_t)std::max(1, env_int("OEQ_B200_PIPELINE_BLOCK_MB", 1024)) << 20;
        const long long min_block = std::max<long long>(recv_min_block_edges(), (long long)(min_block_bytes / row));
        const bool pipelined = k.map.helper_warps > 0 && edges >= 4 * min_block;
        if (pipelined) {
            const long long half = (long long)(workspace_bytes / row / 2);
            long long be = std::min<long long>(half, (edges + 3) / 4);
            be = std::max<long long>(be, std::min<long long>(half, min_block));
            if (be >= 1) {
                char* halves[2] = {(char*)workspace, (char*)workspace + (size_t)half * row};
                long long prev_e0 = -1, prev_n = 0;
                int b = 0;
                for (long long e0 = 0; e0 < edges; e0 += be, ++b) {
                    const long long n = std::min(be, edges - e0);
                    UvuParams prm{};
                    pass1(e0, n, halves[b & 1], prm);
                    if (prev_e0 >= 0) {
                        prm.sum_cols = (const long long*)cols; prm.sum_perm = (const long long*)perm;
                        prm.sum_ws = halves[(b - 1) & 1];
                        prm.sum_items = edges; prm.sum_e_lo = prev_e0; prm.sum_e_hi = prev_e0 + prev_n;
                        prm.sum_first = b == 1; prm.sum_chunk = sum_chunk;
                    }
                    if ((rc = launch_uvu(k, p, prm, st, dx_bulk))) return rc;
                    ++h->last_bwd_launches;
                    prev_e0 = e0; prev_n = n;
                }
                return sum_launch(prev_e0, prev_n, halves[(b - 1) & 1], b == 1);
            }
        }
        bool first = true;
        for (long long e0 = 0; e0 < edges; e0 += block_edges) {
            const long long n = std::min(block_edges, edges - e0);
            UvuParams prm{};
            pass1(e0, n, workspace, prm);
            if ((rc = launch_uvu(k, p, prm, st, dx_bulk))) return rc;
            ++h->last_bwd_launches;
            if ((rc = sum_launch(e0, n, workspace, first))) return rc;
            first = false;
        }
        return OEQ_OK;
    }
    if ((rc = load_kernel(h->bwd, "oeq_uvu_kernel", false))) return rc;
    h->last_bwd_launches = 1;
    UvuParams prm{};
    prm.X = X; prm.Y = Y; prm.W = W; prm.dZ = dZ; prm.dX = dX; prm.dY = dY; prm.dW = dW;
    prm.rows = (const long long*)rows; prm.cols = (const long long*)cols; prm.perm = (const long long*)perm;
    prm.n_items = edges; prm.n_nodes = nodes; prm.status = h->d_status;
#ifdef OEQ_DEV_PROFILE
    if (env_int("OEQ_B200_UVU_PROFILE", 0)) {
        // cycle accounting of CTA 0's first group (development aid): synchronous, prints to stderr
        unsigned long long* d = nullptr;
        OEQ_CUDA(cudaMalloc(&d, 8 * 8));
        OEQ_CUDA(cudaMemsetAsync(d, 0, 8 * 8, st));
        prm.ws = d;
        rc = launch_uvu(h->bwd, p, prm, st, 16);
        unsigned long long hb[8];
        OEQ_CUDA(cudaMemcpyAsync(hb, d, sizeof hb, cudaMemcpyDeviceToHost, st));
        OEQ_CUDA(cudaStreamSynchronize(st));
        cudaFree(d);
        fprintf(stderr, "[oeq_b200 conv backward profile] consumer: cycles %llu waiting for rows %llu items %llu | producer: cycles %llu "
                        "waiting for a stage %llu walking %llu issuing %llu\n", hb[0], hb[1], hb[2], hb[4], hb[5], hb[6], hb[7]);
        return rc;
    }
#endif
    return launch_uvu(h->bwd, p, prm, st);
}

// ---------------------------------------------------------------- second derivatives of the convolution

int oeq_conv_has_double_backward(const oeq_conv* h) {
    return h && h->dbl_state >= 0 && conv_double_backward_supported(h->prob) ? 1 : 0;
}

int oeq_conv_double_backward(oeq_conv* h, int64_t nodes, int64_t edges, const void* X, const void* Y, const void* W,
                             const void* dZ, const void* EX, const void* EY, const void* EW, const int64_t* rows,
                             const int64_t* cols, const int64_t* perm, void* GX, void* GY, void* GW, void* GdZ,
                             void* workspace, size_t workspace_bytes, void* stream) {
    if (!h) return fail(OEQ_ERR_INVALID, "null handle");
    if (nodes < 0 || edges < 0) return fail(OEQ_ERR_INVALID, "negative size");
    if (!oeq_conv_has_double_backward(h)) return fail(OEQ_ERR_UNSUPPORTED, "no fused second derivatives for this problem");
    cudaStream_t st = (cudaStream_t)stream;
    const Problem& p = h->prob;
    if (nodes == 0) return OEQ_OK;
    if (!GX || !GdZ) return fail(OEQ_ERR_INVALID, "null buffer");
    const int e = p.elem();
    if (edges == 0) {
        OEQ_CUDA(cudaMemsetAsync(GX, 0, (size_t)nodes * p.x_dim * e, st));
        OEQ_CUDA(cudaMemsetAsync(GdZ, 0, (size_t)nodes * p.z_dim * e, st));
        return OEQ_OK;
    }
    if (!X || !Y || !W || !dZ || !EX || !EY || !EW || !rows || !cols || !GY || !GW) return fail(OEQ_ERR_INVALID, "null buffer");
    if (h->deterministic && !perm) return fail(OEQ_ERR_INVALID, "deterministic second derivatives need the sender-order permutation");
    const size_t row = recv_row_bytes(p);
    long long block_edges = edges;
    if (h->deterministic) {
        if (!workspace || !aligned16(workspace)) return fail(OEQ_ERR_UNSUPPORTED, "deterministic second derivatives need scratch memory");
        block_edges = (long long)std::min<size_t>(workspace_bytes / row, (size_t)edges);
        if (block_edges < edges && block_edges < recv_min_block_edges())
            return fail(OEQ_ERR_UNSUPPORTED, "deterministic second derivatives need more scratch memory");
    }
    int rc = ensure_status(&h->d_status);
    if (rc) return rc;
    if (h->dbl_state == 0) {
        rc = build_uvu_dblc(p, h->deterministic, false, h->dbl_z);
        if (!rc) rc = build_uvu_dblc(p, h->deterministic, true, h->dbl_g);
        if (!rc) rc = load_kernel(h->dbl_z, "oeq_uvu_kernel", false);
        if (!rc) rc = load_kernel(h->dbl_g, "oeq_uvu_kernel", false);
        if (!rc) {
            OEQ_CUDA(cudaLibraryGetKernel(&h->dbl_sum_fn, h->dbl_g.lib, "oeq_sum_sender_rows"));
            OEQ_CUDA(cudaLibraryGetKernel(&h->dbl_clear_fn, h->dbl_g.lib, "oeq_clear"));
        }
        h->dbl_state = rc ? -1 : 1;
        if (rc) return rc;
    }
    h->last_stream = st;
    // bulk copies of a kind of row only when the row and its cotangent row both qualify
    int clear = 0;
    if (!aligned16(EX)) clear |= 1;
    if (!aligned16(EY)) clear |= 2;
    if (!aligned16(EW)) clear |= 4;
    // gradient with respect to dZ: the forward walk over all edges
    if (!h->deterministic) OEQ_CUDA(cudaMemsetAsync(GdZ, 0, (size_t)nodes * p.z_dim * e, st));
    {
        UvuParams prm{};
        prm.X = X; prm.Y = Y; prm.W = W; prm.Z = GdZ; prm.EX = EX; prm.EY = EY; prm.EW = EW;
        prm.rows = (const long long*)rows; prm.cols = (const long long*)cols;
        prm.n_items = edges; prm.n_nodes = nodes; prm.status = h->d_status;
        if ((rc = launch_uvu(h->dbl_z, p, prm, st, 0, 0, nullptr, clear))) return rc;
    }
    // gradients with respect to X, Y, W: the receiver-order walk, GX through scratch rows or bulk reductions
    Kernel& k = h->dbl_g;
    {
        unsigned long long words = (unsigned long long)nodes * p.x_dim * e / 4;
        void* ptr = GX;
        void* args[] = {&ptr, &words};
        const unsigned grid = (unsigned)std::max<unsigned long long>(1, std::min<unsigned long long>((unsigned long long)k.sm_count * 8, (words / 4 + 255) / 256));
        OEQ_CUDA(cudaLaunchKernel((const void*)h->dbl_clear_fn, dim3(grid), dim3(256), args, 0, st));
    }
    const int dx_bulk = ((p.x_dim * e) % 16 == 0 && aligned16(GX)) ? 32 : 0;
    const int sum_chunk = std::max(1, env_int("OEQ_B200_SUM_CHUNK", 64));
    bool first = true;
    for (long long e0 = 0; e0 < edges; e0 += block_edges) {
        const long long n = std::min(block_edges, edges - e0);
        const size_t yo = (size_t)e0 * p.y_dim * e, wo = (size_t)e0 * p.w_numel * e;
        UvuParams prm{};
        prm.X = X; prm.dZ = dZ; prm.dX = GX; prm.EX = EX;
        prm.Y = (const char*)Y + yo; prm.W = (const char*)W + wo;
        prm.EY = (const char*)EY + yo; prm.EW = (const char*)EW + wo;
        prm.dY = (char*)GY + yo; prm.dW = (char*)GW + wo;
        prm.rows = (const long long*)rows + e0; prm.cols = (const long long*)cols + e0;
        prm.n_items = n; prm.n_nodes = nodes; prm.status = h->d_status;
        prm.ws = h->deterministic ? workspace : nullptr;
        if ((rc = launch_uvu(k, p, prm, st, dx_bulk, 0, nullptr, clear))) return rc;
        if (h->deterministic) {
            UvuParams sp{};
            sp.dX = GX; sp.ws = workspace;
            sp.rows = (const long long*)rows; sp.cols = (const long long*)cols; sp.perm = (const long long*)perm;
            sp.n_items = edges; sp.n_nodes = nodes; sp.status = h->d_status;
            sp.flags = first ? 64 : 0;
            sp.chunk = sum_chunk;
            sp.e_lo = e0; sp.e_hi = e0 + n;
            const long long chunks = (edges + sp.chunk - 1) / sp.chunk;
            const long long grid = std::max<long long>(1, std::min<long long>((long long)k.sm_count * 6, (chunks + 7) / 8));
            void* args[] = {&sp};
            OEQ_CUDA(cudaLaunchKernel((const void*)h->dbl_sum_fn, dim3((unsigned)grid), dim3(256), args, 0, st));
            first = false;
        }
    }
    return OEQ_OK;
}

// ---------------------------------------------------------------- self-test of the bounded waits

// One thread waits on a shared-memory barrier that nothing ever completes, polls `polls` times, gives up, records
// the code in *status and returns: the path every staged kernel takes when a copy never lands.
__global__ void oeq_wait_probe_kernel(int* status, unsigned polls) {
    __shared__ unsigned long long bar;
    if (threadIdx.x == 0) {
        oeq::mbar_init(&bar, 1);
        oeq::fence_mbar_init();
        bool done = false;
        for (unsigned spin = 0; spin < polls && !done; ++spin) done = oeq::mbar_try_wait(&bar, 0u);
        if (!done) atomicCAS(status, 0, oeq::ERR_WAIT_FULL);
    }
}

int oeq_selftest_bounded_wait(int polls, void* stream) {
    if (polls < 1 || polls > (1 << 20)) return fail(OEQ_ERR_INVALID, "polls must be in 1 .. 2^20");
    int* d_status = nullptr;
    int rc = ensure_status(&d_status);
    if (rc) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    oeq_wait_probe_kernel<<<1, 32, 0, st>>>(d_status, (unsigned)polls);
    cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) rc = check_status(d_status, st);      // OEQ_ERR_DEVICE_WAIT is the expected answer
    cudaFree(d_status);
    if (e != cudaSuccess) return fail(OEQ_ERR_CUDA, std::string("wait probe: ") + cudaGetErrorString(e));
    return rc;
}

int oeq_conv_last_backward_launches(const oeq_conv* h) { return h ? h->last_bwd_launches : 0; }

int oeq_conv_check(oeq_conv* h) { return h ? check_status(h->d_status, h->last_stream) : fail(OEQ_ERR_INVALID, "null handle"); }

int oeq_conv_launch_info(const oeq_conv* h, int which, int* threads, int* ng, int* ps, int* stages, int* smem, int* regs) {
    if (!h) return fail(OEQ_ERR_INVALID, "null handle");
    if (which) return launch_info(h->has_bwd_recv && h->bwd_recv.loaded ? h->bwd_recv : h->bwd, threads, ng, ps, stages, smem, regs);
    return launch_info(h->has_fwd_tc && h->fwd_tc.loaded ? h->fwd_tc : h->fwd, threads, ng, ps, stages, smem, regs);
}

}  // extern "C"
