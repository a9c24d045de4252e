// libhemmer_b200.so -- implementation of the C ABI in include/hemmer_b200.h.
// Host code here only plans launches and owns device memory; every residue is computed by the
// sm_100a kernels in ntt.cuh / kernels.cuh.  There is no CPU fallback: without a device the
// context cannot be created.
#include "../../include/hemmer_b200.h"
#include "host_ctx.hpp"
#include "kernels.cuh"
#include "ntt.cuh"

#include <cstdio>
#include <dlfcn.h>
#include <map>
#include <thread>
#include <memory>
#include <mutex>
#include <nccl.h> // types only: the library is resolved at run time, see nccl_api()
#include <unordered_map>

using namespace hb;
using hbhost::HostCtx;
using hbhost::HostParams;

namespace {

struct CudaFail { cudaError_t e; const char *where; };
#define CK(x) do { cudaError_t e__ = (x); if (e__ != cudaSuccess) throw CudaFail{e__, #x}; } while (0)
struct ArgFail { int code; std::string msg; };
[[noreturn]] void fail(int code, const std::string &m) { throw ArgFail{code, m}; }

// Size-bucketed caching allocator: the matmul schedules allocate and free the same few buffer
// sizes thousands of times; cudaMalloc is reached only the first time a size is seen.
struct Pool {
    std::unordered_map<size_t, std::vector<void *>> free_;
    std::unordered_map<void *, size_t> live_;
    size_t total = 0, in_use = 0;
    void *get(size_t bytes) {
        bytes = (bytes + 255) & ~(size_t)255;
        auto &v = free_[bytes];
        void *p = nullptr;
        if (!v.empty()) { p = v.back(); v.pop_back(); }
        else {
            cudaError_t e = cudaMalloc(&p, bytes);
            if (e != cudaSuccess) { release_cached(); e = cudaMalloc(&p, bytes); }
            if (e != cudaSuccess) { cudaGetLastError(); fail(HB_E_OOM, "device allocation of " + std::to_string(bytes) + " bytes failed"); }
            total += bytes;
        }
        live_[p] = bytes; in_use += bytes;
        return p;
    }
    void put(void *p) {
        if (!p) return;
        auto it = live_.find(p);
        if (it == live_.end()) return;
        free_[it->second].push_back(p); in_use -= it->second; live_.erase(it);
    }
    void release_cached() {
        for (auto &kv : free_) { for (void *p : kv.second) { cudaFree(p); total -= kv.first; } kv.second.clear(); }
    }
    ~Pool() { release_cached(); for (auto &kv : live_) cudaFree(kv.first); }
};

struct Evk { u64 *d = nullptr; int nd = 0; };

// NCCL is bound at first use instead of at link time: a process that also loads PyTorch must use the
// NCCL build PyTorch brought along, whichever library was loaded first.
struct NcclApi {
    ncclResult_t (*AllReduce)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllGather)(const void *, void *, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*Reduce)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*Send)(const void *, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*Recv)(void *, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*GroupStart)() = nullptr;
    ncclResult_t (*GroupEnd)() = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    const char *(*GetErrorString)(ncclResult_t) = nullptr;
    bool ok = false;
};
const NcclApi &nccl_api() {
    static NcclApi api = [] {
        NcclApi a;
        void *h = dlsym(RTLD_DEFAULT, "ncclAllReduce") ? RTLD_DEFAULT : dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!h && !dlsym(RTLD_DEFAULT, "ncclAllReduce")) return a;
        auto sym = [&](const char *n) { void *p = dlsym(RTLD_DEFAULT, n); return p ? p : (h && h != RTLD_DEFAULT ? dlsym(h, n) : nullptr); };
        a.AllReduce = (decltype(a.AllReduce))sym("ncclAllReduce");
        a.AllGather = (decltype(a.AllGather))sym("ncclAllGather");
        a.Reduce = (decltype(a.Reduce))sym("ncclReduce");
        a.Send = (decltype(a.Send))sym("ncclSend");
        a.Recv = (decltype(a.Recv))sym("ncclRecv");
        a.GroupStart = (decltype(a.GroupStart))sym("ncclGroupStart");
        a.GroupEnd = (decltype(a.GroupEnd))sym("ncclGroupEnd");
        a.GetUniqueId = (decltype(a.GetUniqueId))sym("ncclGetUniqueId");
        a.CommInitRank = (decltype(a.CommInitRank))sym("ncclCommInitRank");
        a.CommDestroy = (decltype(a.CommDestroy))sym("ncclCommDestroy");
        a.GetErrorString = (decltype(a.GetErrorString))sym("ncclGetErrorString");
        a.ok = a.AllReduce && a.AllGather && a.Reduce && a.Send && a.Recv && a.GroupStart && a.GroupEnd && a.GetUniqueId && a.CommInitRank && a.CommDestroy &&
               a.GetErrorString;
        return a;
    }();
    return api;
}

} // namespace

struct hb_ctx {
    std::unique_ptr<HostCtx> h;
    int device = 0;
    cudaStream_t st = nullptr;
    Pool pool;
    std::string err;
    PrimeConst *pc = nullptr;
    u64 *tw = nullptr; // twiddle tables: psi | psi_sh | ipsi | ipsi_sh, each [nprimes][N], or the 2^16 layout of ntt16.cuh
    NttTables tb{};
    u64 *sk = nullptr; // [nprimes][N] NTT form
    bool have_sk = false;
    Evk mult_key;
    std::map<u64, Evk> gal_keys;
    std::map<int, KsPlan *> plans; // device copies
    std::map<int, DivPlan *> div_plans;
    std::map<int, std::vector<u64>> div_hat_inv; // host copy of DivPlan::hat_inv per level (folded into the inverse transform)
    u64 *pinned = nullptr; size_t pinned_bytes = 0; // host staging buffer of hb_decrypt_many
    ChaChaKey ckey{};
    std::map<std::pair<int, long long>, u32 *> gal_tables; // (copies, row_step) -> Galois elements of hb_matmul_acc, on the device
    int host_threads = 0;                                 // cap for the host-side encode / decode workers (0: all cores, at most 32)
    bool capturing = false;                               // between hb_graph_begin and hb_graph_end
    unsigned long long launches_at_capture = 0, alg_at_capture = 0;
    int N = 0, logn = 0, L = 0, K = 0, nprimes = 0;
    unsigned long long launches = 0; // kernels launched by this context
    int *dev_err = nullptr;          // raised by a kernel whose bounded wait ran out; read by hb_sync
    bool smem_opt_in_mkb = false, smem_opt_in_parts = false; // the opt-in to more than 48 KB of shared memory is per kernel and per device: once per context
    // Compulsory HBM traffic of the primitives called so far, in limbs of N words: every input of a primitive read once,
    // every output written once, a switching key or plaintext once per batch (temporaries and transforms inside a
    // primitive do not count).  Divided by the HBM peak this is the time the call sequence cannot go below.
    unsigned long long alg_limbs = 0;

    LimbMap qmap(int level) const { LimbMap m{}; m.n = level + 1; for (int i = 0; i <= level; ++i) m.prime[i] = (unsigned char)i; return m; }
    LimbMap allmap() const { LimbMap m{}; m.n = nprimes; for (int i = 0; i < nprimes; ++i) m.prime[i] = (unsigned char)i; return m; }
    unsigned gx() const { return (unsigned)((N + 256 * kElems - 1) / (256 * kElems)); } // blocks per limb of the element-wise kernels
    dim3 egrid(int count) const { return dim3(gx(), (unsigned)count); }
    u64 *alloc_limbs(size_t limbs) { return (u64 *)pool.get(limbs * (size_t)N * 8); }
};

#define LAUNCH(c) ((c)->launches++, 0)
#define ALG(c, limbs) ((c)->alg_limbs += (unsigned long long)(limbs))
struct hb_ct { hb_ctx *ctx; int level, np, batch, spow; u64 *d; size_t limbs() const { return (size_t)batch * np * (level + 1); } };
struct hb_pt { hb_ctx *ctx; int level, spow; u64 *d; int ext = 0; }; // ext: K further limbs modulo the special primes follow the level+1 limbs
// lifted digits of the a-part of a ciphertext batch, NTT form: what all rotations of that ciphertext share
struct hb_digits { hb_ctx *ctx; int level, batch; u64 *d; };
// a switching key multiplied by a plaintext mask, restricted to one level: key [nd][2][ne][N], pm = P * mask on the Q limbs [n][N]
struct hb_mkey { hb_ctx *ctx; int level; u32 g; u64 *key, *pm; };

namespace {

// entry points that wait for the stream or copy to / from the host cannot be part of a recorded graph
void no_capture(const hb_ctx *c, const char *what) { if (c->capturing) fail(HB_E_ARG, std::string(what) + ": not available while a graph is being recorded"); }
// A handle is only valid with the context that made it: its buffer lives in that context's pool, on that
// context's device.
template <class H> void own1(const hb_ctx *c, const H *h) { if (h && h->ctx != c) fail(HB_E_ARG, "handle belongs to another context"); }
template <class... H> void own(const hb_ctx *c, const H *...h) { (own1(c, h), ...); }

hb_ct *new_ct(hb_ctx *c, int level, int np, int batch, int spow) {
    if (level < 0 || level > c->L || np < 1 || np > 3 || batch < 1 || spow < 1 || spow > 2) fail(HB_E_ARG, "bad ciphertext geometry");
    hb_ct *x = new hb_ct{c, level, np, batch, spow, nullptr};
    try { x->d = c->alloc_limbs(x->limbs()); } catch (...) { delete x; throw; }
    return x;
}
hb_pt *new_pt(hb_ctx *c, int level, int spow) {
    hb_pt *x = new hb_pt{c, level, spow, nullptr};
    try { x->d = c->alloc_limbs((size_t)level + 1); } catch (...) { delete x; throw; }
    return x;
}
struct Tmp { // pool buffer released at scope exit
    hb_ctx *c; u64 *p;
    Tmp(hb_ctx *cc, size_t limbs) : c(cc), p(cc->alloc_limbs(limbs)) {}
    ~Tmp() { c->pool.put(p); }
    Tmp(const Tmp &) = delete;
};

struct TmpBytes { // the same for a byte count (staging buffers of int64 coefficients)
    hb_ctx *c; void *p;
    TmpBytes(hb_ctx *cc, size_t bytes) : c(cc), p(cc->pool.get(bytes)) {}
    ~TmpBytes() { c->pool.put(p); }
    TmpBytes(const TmpBytes &) = delete;
};

void ntt(hb_ctx *c, const u64 *src, size_t so, u64 *dst, size_t dof, int count, const LimbMap &m, bool inv, const Ntt16Scale *scale = nullptr) {
    c->launches += (count == 0) ? 0 : (c->logn == 16 ? 2 : 1);
    CK(launch_ntt(c->st, src, so, dst, dof, count, m, c->pc, c->tb, c->logn, inv, scale));
}
// scale table of an inverse transform that also multiplies position k by f[k] (2^16 rings only): s_k = N^-1 * f[k] mod q
Ntt16Scale ntt_scale(hb_ctx *c, const LimbMap &m, const u64 *f) {
    Ntt16Scale sc{};
    if (m.n > 8) fail(HB_E_LIMIT, "scaled inverse transform: at most 8 limb positions");
    sc.on = 1;
    for (int k = 0; k < m.n; ++k) {
        const u64 q = c->h->q[m.prime[k]];
        const u64 s = hbhost::mulmod(hbhost::invmod((u64)c->N % q, q), f[k] % q, q);
        if (q >> 44) { sc.w[k] = s; sc.comp[k] = hbhost::shoup(s, q); }
        else {
            sc.w[k] = ds_twiddle_word(s);
            const double sf = (double)s / (double)q;
            std::memcpy(&sc.comp[k], &sf, 8);
        }
    }
    return sc;
}
void ntt_inplace(hb_ctx *c, u64 *d, int count, const LimbMap &m, bool inv) { ntt(c, d, (size_t)m.n * c->N, d, (size_t)m.n * c->N, count, m, inv); }

// ---- key-switch plan for one level ----
const KsPlan *get_plan(hb_ctx *c, int level) {
    auto it = c->plans.find(level);
    if (it != c->plans.end()) return it->second;
    no_capture(c, "first key switch at this level");
    const HostCtx &h = *c->h;
    auto P = std::make_unique<KsPlan>();
    std::memset(P.get(), 0, sizeof(KsPlan));
    const int n = level + 1, K = h.K, ne = n + K;
    P->level = level; P->n = n; P->ne = ne; P->K = K; P->nd = h.digit_of(level) + 1;
    for (int j = 0; j < ne; ++j) P->ext_prime[j] = (unsigned char)(j < n ? j : h.L + 1 + (j - n));
    int entry = 0;
    for (int dg = 0; dg < P->nd; ++dg) {
        const int lo = h.digit_lo(dg), hi = h.digit_hi(dg, n), ns = hi - lo;
        P->dig_lo[dg] = lo; P->dig_hi[dg] = hi; P->dt_start[dg] = entry;
        for (int s = 0; s < ns; ++s) {
            const u64 qs = h.q[lo + s];
            u64 hat = 1;
            for (int t = 0; t < ns; ++t) if (t != s) hat = hbhost::mulmod(hat, h.q[lo + t] % qs, qs);
            u64 hi_ = hbhost::invmod(hat, qs);
            P->hat_inv[dg][s] = hi_; P->hat_inv_sh[dg][s] = hbhost::shoup(hi_, qs);
            for (int j = 0; j < ne; ++j) {
                const u64 qt = h.q[P->ext_prime[j]];
                u64 hm = 1;
                for (int t = 0; t < ns; ++t) if (t != s) hm = hbhost::mulmod(hm, h.q[lo + t] % qt, qt);
                P->hat_mod[dg][s][j] = hm;
                const double d0 = (double)hm, d1 = (double)hbhost::mulmod(hm, ((u64)1 << 30) % qt, qt);
                std::memcpy(&P->hat_mod_d0[dg][s][j], &d0, 8);
                std::memcpy(&P->hat_mod_d1[dg][s][j], &d1, 8);
            }
        }
        for (int j = 0; j < ne; ++j) {
            if (j >= lo && j < hi) P->dt_entry[dg][j] = -1;
            else P->dt_entry[dg][j] = (short)entry++;
        }
    }
    P->dt_count = entry;
    for (int k = 0; k < K; ++k) {
        const u64 pk = h.q[h.L + 1 + k];
        u64 hat = 1;
        for (int t = 0; t < K; ++t) if (t != k) hat = hbhost::mulmod(hat, h.q[h.L + 1 + t] % pk, pk);
        u64 hi_ = hbhost::invmod(hat, pk);
        P->p_hat_inv[k] = hi_; P->p_hat_inv_sh[k] = hbhost::shoup(hi_, pk);
        for (int l = 0; l < n; ++l) {
            const u64 ql = h.q[l];
            u64 hm = 1;
            for (int t = 0; t < K; ++t) if (t != k) hm = hbhost::mulmod(hm, h.q[h.L + 1 + t] % ql, ql);
            P->p_hat_mod[k][l] = hm;
            const double d0 = (double)hm, d1 = (double)hbhost::mulmod(hm, ((u64)1 << 30) % ql, ql);
            std::memcpy(&P->p_hat_mod_d0[k][l], &d0, 8);
            std::memcpy(&P->p_hat_mod_d1[k][l], &d1, 8);
        }
    }
    for (int l = 0; l < n; ++l) {
        const u64 ql = h.q[l];
        u64 pm = 1;
        for (int t = 0; t < K; ++t) pm = hbhost::mulmod(pm, h.q[h.L + 1 + t] % ql, ql);
        P->p_inv[l] = hbhost::invmod(pm, ql);
    }
    KsPlan *d = nullptr;
    CK(cudaMalloc(&d, sizeof(KsPlan)));
    CK(cudaMemcpyAsync(d, P.get(), sizeof(KsPlan), cudaMemcpyHostToDevice, c->st));
    CK(cudaStreamSynchronize(c->st));
    c->plans[level] = d;
    return d;
}
// host mirror of the few plan fields the launcher needs
struct PlanDims { int n, ne, nd, K, dt_count; LimbMap dtmap; };
PlanDims plan_dims(hb_ctx *c, int level) {
    const HostCtx &h = *c->h;
    PlanDims p{}; p.n = level + 1; p.K = h.K; p.ne = p.n + h.K; p.nd = h.digit_of(level) + 1;
    int e = 0;
    for (int dg = 0; dg < p.nd; ++dg) {
        const int lo = h.digit_lo(dg), hi = h.digit_hi(dg, p.n);
        for (int j = 0; j < p.ne; ++j) {
            if (j >= lo && j < hi) continue;
            if (e >= kMaxList) fail(HB_E_LIMIT, "too many lifted limbs");
            p.dtmap.prime[e++] = (unsigned char)(j < p.n ? j : h.L + 1 + (j - p.n));
        }
    }
    p.dt_count = e; p.dtmap.n = e;
    return p;
}

size_t key_limbs(hb_ctx *c, int level) { const PlanDims d = plan_dims(c, level); return (size_t)2 * d.nd * d.ne; } // the part of a switching key one key switch reads

// Hybrid key switch of polynomial a (NTT form, `n` limbs, per-batch stride a_outer) with key `key`:
//   out[b][p][l] = ModDown(sum_dg perm_g(lift_dg(a)) (.) key_dg)[p][l] + add_p[b][l] o perm_g
// Phase 1 of a key switch (shared by every rotation of the same polynomial -- "hoisting"):
//   dt[b][entry] = NTT(lift of digit dg of a to ext limb j), for the limbs outside the digit.
void ks_decompose(hb_ctx *c, const u64 *a, size_t a_outer, int level, int batch, u64 *dt) {
    const KsPlan *pl = get_plan(c, level);
    const PlanDims d = plan_dims(c, level);
    const int N = c->N, n = d.n;
    const unsigned gx1 = (unsigned)((N + 255) / 256); // base-conversion kernels keep one coefficient per thread
    Tmp acoef(c, (size_t)batch * n);
    ntt(c, a, a_outer, acoef.p, (size_t)n * N, batch * n, c->qmap(level), true);
    LAUNCH(c), k_modup<<<dim3(gx1, d.nd, batch), 256, 0, c->st>>>(dt, acoef.p, pl, c->pc, N);
    ntt_inplace(c, dt, batch * d.dt_count, d.dtmap, false);
}
// ModDown of acc [batch*2][ne][N] into out: conversion of the special limbs, forward transform, final combination
void moddown(hb_ctx *c, const u64 *acc, u64 *pco, u64 *tbuf, int level, int batch, u64 *out, size_t out_outer, const u64 *add0, const u64 *add1, size_t add_outer, u32 g) {
    const KsPlan *pl = get_plan(c, level);
    const PlanDims d = plan_dims(c, level);
    const int N = c->N, n = d.n, ne = d.ne, K = d.K;
    const unsigned gx1 = (unsigned)((N + 255) / 256), gx = c->gx();
    LimbMap pm{}; pm.n = K; for (int k = 0; k < K; ++k) pm.prime[k] = (unsigned char)(c->L + 1 + k);
    ntt(c, acc + (size_t)n * N, (size_t)ne * N, pco, (size_t)K * N, batch * 2 * K, pm, true);
    LAUNCH(c), k_moddown_conv<<<dim3(gx1, 1, batch * 2), 256, 0, c->st>>>(tbuf, pco, pl, c->pc, c->L + 1, N);
    ntt_inplace(c, tbuf, batch * 2 * n, c->qmap(level), false);
    LAUNCH(c), k_moddown_fin<<<dim3(gx, n, batch * 2), 256, 0, c->st>>>(out, out_outer, acc, tbuf, add0, add1, add_outer, pl, c->pc, g, c->logn, N);
    CK(cudaGetLastError());
}
// Phase 2: inner product of the (permuted) digits with the key over Q_level u P, then ModDown:
//   out[b][p][l] = ModDown(sum_dg perm_g(digit_dg) (.) key_dg)[p][l] + add_p[b][l] o perm_g
void ks_apply(hb_ctx *c, const u64 *a, size_t a_outer, const u64 *dt, int level, int batch, const Evk &key, u32 g, u64 *out, size_t out_outer, const u64 *add0,
              const u64 *add1, size_t add_outer) {
    const KsPlan *pl = get_plan(c, level);
    const PlanDims d = plan_dims(c, level);
    const int N = c->N, n = d.n, ne = d.ne, K = d.K;
    const unsigned gx = c->gx();
    Tmp acc(c, (size_t)batch * 2 * ne), pco(c, (size_t)batch * 2 * K), t(c, (size_t)batch * 2 * n);
    LAUNCH(c), k_ks_inner<<<dim3(gx, batch, ne), 256, 0, c->st>>>(acc.p, a, a_outer, dt, key.d, c->nprimes, pl, c->pc, g, c->logn, N);
    moddown(c, acc.p, pco.p, t.p, level, batch, out, out_outer, add0, add1, add_outer, g);
}
// Hybrid key switch of polynomial a (NTT form, `n` limbs, per-batch stride a_outer) with key `key`
void keyswitch(hb_ctx *c, const u64 *a, size_t a_outer, int level, int batch, const Evk &key, u32 g, u64 *out, size_t out_outer, const u64 *add0, const u64 *add1,
               size_t add_outer) {
    const PlanDims d = plan_dims(c, level);
    Tmp dt(c, (size_t)batch * d.dt_count);
    ks_decompose(c, a, a_outer, level, batch, dt.p);
    ks_apply(c, a, a_outer, dt.p, level, batch, key, g, out, out_outer, add0, add1, add_outer);
}

// Galois elements of the row shifts k * row_step, k < copies, kept on the device per (copies, row_step): the fused
// plaintext-matmul accumulate reads them on every call, and a per-call upload would need a host synchronisation.
const u32 *galois_table(hb_ctx *c, int copies, i64 row_step) {
    const auto key = std::make_pair(copies, (long long)row_step);
    auto it = c->gal_tables.find(key);
    if (it != c->gal_tables.end()) return it->second;
    if (c->capturing) fail(HB_E_ARG, "matmul_acc: first use of this (copies, row_step) pair inside a graph capture; run the step once before capturing");
    std::vector<u32> gal((size_t)copies);
    for (int k = 0; k < copies; ++k) gal[(size_t)k] = (u32)c->h->galois_rot((i64)k * row_step);
    u32 *d = nullptr;
    CK(cudaMalloc(&d, (size_t)copies * 4));
    cudaError_t e = cudaMemcpyAsync(d, gal.data(), (size_t)copies * 4, cudaMemcpyHostToDevice, c->st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(c->st); // gal goes out of scope
    if (e != cudaSuccess) { cudaFree(d); throw CudaFail{e, "galois_table upload"}; }
    c->gal_tables[key] = d;
    return d;
}

// switching key for secret s' (g == 0: s^2, else s o perm_g); stream ids kid*64 + digit
Evk make_key(hb_ctx *c, u64 kid, u32 g) {
    if (!c->have_sk) fail(HB_E_NOKEY, "secret key not generated");
    no_capture(c, "key generation");
    const HostCtx &h = *c->h;
    const int N = c->N, np = c->nprimes, nd = h.digit_of(h.L) + 1;
    Evk k; k.nd = nd; k.d = c->alloc_limbs((size_t)nd * 2 * np);
    const LimbMap am = c->allmap();
    Tmp e(c, (size_t)np);
    TmpBytes ecoef_buf(c, (size_t)N * 8);
    i64 *ecoef = (i64 *)ecoef_buf.p;
    Scalars pmod{};
    for (int pi = 0; pi <= h.L; ++pi) { u64 v = 1; for (int j = 0; j < h.K; ++j) v = hbhost::mulmod(v, h.q[h.L + 1 + j] % h.q[pi], h.q[pi]); pmod.v[pi] = v; }
    std::vector<i64> ev;
    for (int dg = 0; dg < nd; ++dg) {
        u64 *b = k.d + ((size_t)dg * 2) * np * N, *a = b + (size_t)np * N;
        LAUNCH(c), k_uniform<<<dim3((unsigned)((N / 4 + 255) / 256), np), 256, 0, c->st>>>(a, am, c->pc, N, c->ckey, hbhost::STREAM_KEY_A, kid * 64 + dg);
        h.sample_gauss(hbhost::STREAM_KEY_E, kid * 64 + dg, ev);
        CK(cudaMemcpyAsync(ecoef, ev.data(), (size_t)N * 8, cudaMemcpyHostToDevice, c->st));
        LAUNCH(c), k_reduce_i64<<<c->egrid(np), 256, 0, c->st>>>(e.p, ecoef, am, c->pc, N);
        CK(cudaStreamSynchronize(c->st)); // ev is reused by the next digit
        ntt_inplace(c, e.p, np, am, false);
        LAUNCH(c), k_keygen<<<c->egrid(np), 256, 0, c->st>>>(b, a, e.p, c->sk, c->pc, N, c->logn, g, h.digit_lo(dg), h.digit_hi(dg, h.L + 1), pmod);
    }
    CK(cudaGetLastError());
    return k;
}
const Evk &galois_key(hb_ctx *c, u64 g) {
    auto it = c->gal_keys.find(g);
    if (it == c->gal_keys.end()) fail(HB_E_NOKEY, "no switching key for galois element " + std::to_string(g));
    return it->second;
}

// ---- division of a Q_level u P polynomial by P * q_level (masked pair of rotations) ----
const DivPlan *get_div_plan(hb_ctx *c, int level) {
    auto it = c->div_plans.find(level);
    if (it != c->div_plans.end()) return it->second;
    no_capture(c, "first masked rotation at this level");
    const HostCtx &h = *c->h;
    auto P = std::make_unique<DivPlan>();
    std::memset(P.get(), 0, sizeof(DivPlan));
    const int K = h.K, ns = K + 1;
    if (ns > 8) fail(HB_E_LIMIT, "too many special primes");
    P->level = level; P->ns = ns;
    P->src_prime[0] = (unsigned char)level;
    for (int k = 0; k < K; ++k) P->src_prime[1 + k] = (unsigned char)(h.L + 1 + k);
    for (int s = 0; s < ns; ++s) {
        const u64 ds = h.q[P->src_prime[s]];
        u64 hat = 1;
        for (int t = 0; t < ns; ++t) if (t != s) hat = hbhost::mulmod(hat, h.q[P->src_prime[t]] % ds, ds);
        const u64 hi_ = hbhost::invmod(hat, ds);
        P->hat_inv[s] = hi_; P->hat_inv_sh[s] = hbhost::shoup(hi_, ds);
        c->div_hat_inv[level].push_back(hi_);
        for (int l = 0; l < level; ++l) {
            const u64 ql = h.q[l];
            u64 hm = 1;
            for (int t = 0; t < ns; ++t) if (t != s) hm = hbhost::mulmod(hm, h.q[P->src_prime[t]] % ql, ql);
            P->hat_mod[s][l] = hm;
            const double d0 = (double)hm, d1 = (double)hbhost::mulmod(hm, ((u64)1 << 30) % ql, ql);
            std::memcpy(&P->hat_mod_d0[s][l], &d0, 8);
            std::memcpy(&P->hat_mod_d1[s][l], &d1, 8);
        }
    }
    for (int l = 0; l <= level; ++l) {
        const u64 ql = h.q[l];
        u64 pm = 1;
        for (int k = 0; k < K; ++k) pm = hbhost::mulmod(pm, h.q[h.L + 1 + k] % ql, ql);
        P->p_mod[l] = pm;
        if (l < level) P->d_inv[l] = hbhost::invmod(hbhost::mulmod(pm, h.q[level] % ql, ql), ql);
    }
    DivPlan *d = nullptr;
    CK(cudaMalloc(&d, sizeof(DivPlan)));
    CK(cudaMemcpyAsync(d, P.get(), sizeof(DivPlan), cudaMemcpyHostToDevice, c->st));
    CK(cudaStreamSynchronize(c->st));
    c->div_plans[level] = d;
    return d;
}
// E [batch][2][ne][N] over Q_level u P  ->  new ciphertext at level - 1:  (E - lift(E mod P*q_level)) / (P*q_level)
hb_ct *divide_by_p_ql(hb_ctx *c, const u64 *E, int level, int batch) {
    const DivPlan *dv = get_div_plan(c, level);
    const PlanDims d = plan_dims(c, level);
    const int N = c->N, n = d.n, ne = d.ne, ns = d.K + 1;
    hb_ct *r = new_ct(c, level - 1, 2, batch, 1);
    try {
        const unsigned gx1 = (unsigned)((N + 255) / 256), gx = c->gx();
        Tmp sc(c, (size_t)batch * 2 * ns), t(c, (size_t)batch * 2 * level);
        LimbMap sm{}; sm.n = ns; sm.prime[0] = (unsigned char)level; for (int k = 0; k < d.K; ++k) sm.prime[1 + k] = (unsigned char)(c->L + 1 + k);
        // 2^16 rings: the inverse transform multiplies limb s by (D / d_s)^-1 on its way out, the conversion starts from there
        const bool fold = c->logn == 16;
        if (fold) {
            const Ntt16Scale scale = ntt_scale(c, sm, c->div_hat_inv[level].data());
            ntt(c, E + (size_t)(n - 1) * N, (size_t)ne * N, sc.p, (size_t)ns * N, batch * 2 * ns, sm, true, &scale);
        } else ntt(c, E + (size_t)(n - 1) * N, (size_t)ne * N, sc.p, (size_t)ns * N, batch * 2 * ns, sm, true);
        LAUNCH(c), k_div_conv<<<dim3(gx1, 1, batch * 2), 256, 0, c->st>>>(t.p, sc.p, dv, c->pc, N, fold ? 1 : 0);
        ntt_inplace(c, t.p, batch * 2 * level, c->qmap(level - 1), false);
        LAUNCH(c), k_div_fin<<<dim3(gx, level, batch * 2), 256, 0, c->st>>>(r->d, E, t.p, ne, dv, c->pc, N);
        CK(cudaGetLastError());
    } catch (...) { hb_ct_free(r); throw; }
    return r;
}
// rescale(p1 (.) rot(a, s1) + p2 (.) rot(a, s2)) from the lifted digits `dt` of a: both inner products stay in
// Q_level u P, are multiplied there by the extended plaintexts and summed; one division by P * q_level follows.
hb_ct *do_assemble_rot(hb_ctx *c, const hb_ct *a, const u64 *dt, int64_t s1, const hb_pt *p1, int64_t s2, const hb_pt *p2) {
    own(c, a); own(c, p1, p2);
    if (a->np != 2 || a->spow != 1) fail(HB_E_SHAPE, "assemble_rot: needs a rescaled 2-poly ciphertext");
    if (a->level < 1) fail(HB_E_LEVEL, "assemble_rot: level 0");
    if (!p1->ext || !p2->ext || p1->level != a->level || p2->level != a->level || p1->spow != 1 || p2->spow != 1)
        fail(HB_E_LEVEL, "assemble_rot: plaintexts must be extended and at the ciphertext's level");
    const u64 g1 = c->h->galois_rot(s1), g2 = c->h->galois_rot(s2);
    if (g1 == 1 || g2 == 1) fail(HB_E_ARG, "assemble_rot: zero rotation");
    const int level = a->level, batch = a->batch, N = c->N;
    const KsPlan *pl = get_plan(c, level);
    const DivPlan *dv = get_div_plan(c, level);
    const PlanDims d = plan_dims(c, level);
    const int n = d.n, ne = d.ne;
    RotPair rp{};
    rp.key[0] = galois_key(c, g1).d; rp.key[1] = galois_key(c, g2).d;
    rp.mask[0] = p1->d; rp.mask[1] = p2->d;
    rp.g[0] = (u32)g1; rp.g[1] = (u32)g2;
    Tmp E(c, (size_t)batch * 2 * ne);
    ALG(c, (size_t)batch * (2 * n + d.dt_count + 2 * (n - 1)) + 2 * ((size_t)d.nd * 2 * ne + ne));
    const size_t a_outer = (size_t)2 * n * N;
    LAUNCH(c), k_ks_inner_pair<<<dim3(c->gx(), ne, batch), 256, 0, c->st>>>(E.p, a->d, a->d + (size_t)n * N, a_outer, dt, rp, c->nprimes, pl, dv, c->pc, c->logn, N);
    return divide_by_p_ql(c, E.p, level, batch);
}
// the same from keys that already carry the masks (hb_masked_key_create).  `groups` wrapped copies of the same input
// (each with its own one or two keys: k1s[g], k2s[g] or null) come out of one launch sequence, group-major.
hb_ct *do_assemble_mk(hb_ctx *c, const hb_ct *a, const u64 *dt, const hb_mkey *const *k1s, const hb_mkey *const *k2s, int groups) {
    own(c, a);
    if (a->np != 2 || a->spow != 1) fail(HB_E_SHAPE, "assemble: needs a rescaled 2-poly ciphertext");
    if (a->level < 1) fail(HB_E_LEVEL, "assemble: level 0");
    if (groups < 1 || groups > kMaxRotGroups) fail(HB_E_LIMIT, "assemble: 1 to 16 wrapped copies per call");
    MaskedRotList mrl{};
    for (int g = 0; g < groups; ++g) {
        MaskedRot &mr = mrl.r[g];
        const hb_mkey *ks[2] = {k1s[g], k2s ? k2s[g] : nullptr};
        if (!ks[0]) fail(HB_E_ARG, "assemble: missing masked key");
        mr.count = ks[1] ? 2 : 1;
        for (int r = 0; r < mr.count; ++r) {
            if (ks[r]->level != a->level) fail(HB_E_LEVEL, "assemble: masked key of another level");
            own(c, ks[r]);
            mr.mkey[r] = ks[r]->key; mr.pm[r] = ks[r]->pm; mr.g[r] = ks[r]->g;
        }
    }
    const int level = a->level, batch = a->batch, N = c->N;
    const KsPlan *pl = get_plan(c, level);
    const PlanDims d = plan_dims(c, level);
    const int n = d.n, ne = d.ne;
    Tmp E(c, (size_t)groups * batch * 2 * ne);
    for (int g = 0; g < groups; ++g) ALG(c, (size_t)mrl.r[g].count * ((size_t)d.nd * 2 * ne + n) + (size_t)batch * 2 * (n - 1));
    ALG(c, (size_t)batch * (2 * n + d.dt_count));
    // Up to two digits: the bulk-copy kernel (three members per CTA, 512 coefficients; 112 KB of shared memory, two CTAs
    // per SM).  With more digits its staging buffers leave room for one CTA per SM only and the register kernel is faster.
    if (d.nd <= 2 && N % 512 == 0) {
        constexpr int M = 3, EL = 2, T = 256 * EL;
        const int chunks = (batch + M - 1) / M;
        int maxcount = 1;
        for (int g = 0; g < groups; ++g) maxcount = std::max(maxcount, mrl.r[g].count);
        const size_t smem = ((size_t)maxcount * d.nd * 2 + maxcount + (size_t)M * maxcount * (d.nd + 1)) * T * 8;
        if (!c->smem_opt_in_mkb) { CK(cudaFuncSetAttribute(k_ks_inner_mkb<M, EL>, cudaFuncAttributeMaxDynamicSharedMemorySize, 28 * T * 8)); c->smem_opt_in_mkb = true; }
        LAUNCH(c), k_ks_inner_mkb<M, EL><<<dim3((unsigned)(N / T), (unsigned)(groups * chunks), (unsigned)ne), 256, smem, c->st>>>(E.p, a->d, a->d + (size_t)n * N, (size_t)2 * n * N, dt, mrl, batch,
                                                                                                                              maxcount, pl, c->pc, c->logn, N, c->dev_err);
        CK(cudaGetLastError());
        return divide_by_p_ql(c, E.p, level, groups * batch);
    }
    constexpr int kEl = 4; // coefficients per thread (2, with three CTAs resident per SM, measured no faster)
    LAUNCH(c), k_ks_inner_mk<kEl><<<dim3((unsigned)((N + 256 * kEl - 1) / (256 * kEl)), groups * batch, ne), 256, 0, c->st>>>(E.p, a->d, a->d + (size_t)n * N, (size_t)2 * n * N, dt, mrl, batch, pl, c->pc,
                                                                                                                        c->logn, N);
    return divide_by_p_ql(c, E.p, level, groups * batch);
}

void check_same(const hb_ct *a, const hb_ct *b, const char *what) {
    if (a->level != b->level) fail(HB_E_LEVEL, std::string(what) + ": level mismatch");
    if (a->np != b->np || a->batch != b->batch || a->spow != b->spow) fail(HB_E_SHAPE, std::string(what) + ": shape mismatch");
}

hb_ct *do_rescale(hb_ctx *c, const hb_ct *a) {
    own(c, a);
    if (a->level < 1) fail(HB_E_LEVEL, "rescale: level 0");
    if (a->spow != 2) fail(HB_E_SHAPE, "rescale: nothing to rescale");
    const int l = a->level, N = c->N, nbp = a->batch * a->np;
    hb_ct *r = new_ct(c, l - 1, a->np, a->batch, 1);
    ALG(c, (size_t)nbp * (2 * l + 1));
    try {
        Tmp last(c, (size_t)nbp), t(c, (size_t)nbp * l);
        LimbMap lm{}; lm.n = 1; lm.prime[0] = (unsigned char)l;
        ntt(c, a->d + (size_t)l * N, (size_t)(l + 1) * N, last.p, (size_t)N, nbp, lm, true);
        LAUNCH(c), k_rescale_prep<<<c->egrid(nbp * l), 256, 0, c->st>>>(t.p, last.p, l, c->pc, N);
        ntt_inplace(c, t.p, nbp * l, c->qmap(l - 1), false);
        Scalars qi{};
        for (int i = 0; i < l; ++i) qi.v[i] = hbhost::invmod(c->h->q[l] % c->h->q[i], c->h->q[i]);
        LAUNCH(c), k_rescale_fin<<<c->egrid(nbp * l), 256, 0, c->st>>>(r->d, a->d, t.p, l, c->pc, N, qi);
        CK(cudaGetLastError());
    } catch (...) { hb_ct_free(r); throw; }
    return r;
}
// sum_j rescale(a_j (.) p_j)  (separate)  or  rescale(sum_j a_j (.) p_j)
hb_ct *do_prod_rescale(hb_ctx *c, const hb_ct *const *a, const hb_pt *const *p, int count, bool separate) {
    if (count < 1 || count > kMaxTerms) fail(HB_E_LIMIT, "product sum: between 1 and " + std::to_string(kMaxTerms) + " terms");
    const hb_ct *a0 = a[0];
    if (a0->level < 1) fail(HB_E_LEVEL, "rescale: level 0");
    TermList tl{}; tl.count = count;
    for (int j = 0; j < count; ++j) {
        if (a[j]->level != a0->level || p[j]->level != a0->level) fail(HB_E_LEVEL, "mul_pt: level mismatch");
        own(c, a[j]); own(c, p[j]);
        if (a[j]->np != a0->np || a[j]->batch != a0->batch) fail(HB_E_SHAPE, "product sum: shape mismatch");
        if (a[j]->spow != 1 || p[j]->spow != 1) fail(HB_E_SHAPE, "mul_pt: operand not rescaled");
        tl.a[j] = a[j]->d; tl.p[j] = p[j]->d;
    }
    const int l = a0->level, N = c->N, nbp = a0->batch * a0->np, groups = separate ? count : 1;
    const unsigned gx = c->gx();
    hb_ct *r = new_ct(c, l - 1, a0->np, a0->batch, 1);
    ALG(c, (size_t)count * ((size_t)nbp * (l + 1) + (l + 1)) + (size_t)nbp * l);
    try {
        Tmp last(c, (size_t)groups * nbp), S(c, (size_t)nbp), t(c, (size_t)nbp * l);
        LAUNCH(c), k_last_prod<<<dim3(gx, nbp, groups), 256, 0, c->st>>>(last.p, tl, separate ? 1 : 0, l, nbp, c->pc, N);
        LimbMap lm{}; lm.n = 1; lm.prime[0] = (unsigned char)l;
        ntt_inplace(c, last.p, groups * nbp, lm, true);
        LAUNCH(c), k_centre_sum<<<dim3(gx, nbp), 256, 0, c->st>>>((i64 *)S.p, last.p, groups, nbp, l, c->pc, N);
        LAUNCH(c), k_lift_mod<<<c->egrid(nbp * l), 256, 0, c->st>>>(t.p, (const i64 *)S.p, l, c->pc, N);
        ntt_inplace(c, t.p, nbp * l, c->qmap(l - 1), false);
        Scalars qi{};
        for (int i = 0; i < l; ++i) qi.v[i] = hbhost::invmod(c->h->q[l] % c->h->q[i], c->h->q[i]);
        LAUNCH(c), k_prod_rescale_fin<<<c->egrid(nbp * l), 256, 0, c->st>>>(r->d, tl, t.p, l, nbp, c->pc, N, qi);
        CK(cudaGetLastError());
    } catch (...) { hb_ct_free(r); throw; }
    return r;
}
// out_g = rescale(sum_j a_j (.) p[g * count + j]) for every part g in one pass over the a_j; out holds parts * batch members, part-major
hb_ct *do_prod_rescale_parts(hb_ctx *c, const hb_ct *const *a, const hb_pt *const *p, int count, int parts) {
    if (count < 1 || count > kMaxPartTerms || parts < 1 || parts > kMaxParts) fail(HB_E_LIMIT, "product sums: 1 to 17 terms, 1 to 17 parts");
    const hb_ct *a0 = a[0];
    if (!a0) fail(HB_E_ARG, "product sums: null ciphertext");
    if (a0->level < 1) fail(HB_E_LEVEL, "rescale: level 0");
    if (c->N % 256) fail(HB_E_LIMIT, "product sums: ring degree below 256");
    PartTerms pt{}; pt.count = count; pt.parts = parts;
    size_t used = 0;
    for (int j = 0; j < count; ++j) {
        if (!a[j]) fail(HB_E_ARG, "product sums: null ciphertext");
        own(c, a[j]);
        if (a[j]->level != a0->level) fail(HB_E_LEVEL, "mul_pt: level mismatch");
        if (a[j]->np != a0->np || a[j]->batch != a0->batch) fail(HB_E_SHAPE, "product sums: shape mismatch");
        if (a[j]->spow != 1) fail(HB_E_SHAPE, "mul_pt: operand not rescaled");
        pt.a[j] = a[j]->d;
    }
    for (int g = 0; g < parts; ++g) {
        int terms = 0;
        for (int j = 0; j < count; ++j) {
            const hb_pt *q = p[(size_t)g * count + j];
            if (!q) continue;
            own(c, q);
            if (q->level != a0->level) fail(HB_E_LEVEL, "mul_pt: level mismatch");
            if (q->spow != 1) fail(HB_E_SHAPE, "mul_pt: operand not rescaled");
            pt.p[g][j] = q->d; ++terms; ++used;
        }
        if (!terms) fail(HB_E_ARG, "product sums: a part without terms");
    }
    const int l = a0->level, N = c->N, nbp = a0->batch * a0->np, gnbp = parts * nbp;
    const unsigned gx1 = (unsigned)((N + 255) / 256);
    hb_ct *r = new_ct(c, l - 1, a0->np, parts * a0->batch, 1);
    ALG(c, (size_t)count * nbp * (l + 1) + used * (l + 1) + (size_t)gnbp * l);
    try {
        Tmp last(c, (size_t)gnbp), S(c, (size_t)gnbp), t(c, (size_t)gnbp * l);
        constexpr int G = 6; // parts per CTA: 6 x 17 mask chunks of 2 KB = 204 KB of shared memory
        const size_t smem = (size_t)G * count * 2048;
        const unsigned pg = (unsigned)((parts + G - 1) / G);
        if (!c->smem_opt_in_parts) { CK(cudaFuncSetAttribute(k_prod_parts<G>, cudaFuncAttributeMaxDynamicSharedMemorySize, G * kMaxPartTerms * 2048)); c->smem_opt_in_parts = true; }
        Scalars qi{};
        for (int i = 0; i < l; ++i) qi.v[i] = hbhost::invmod(c->h->q[l] % c->h->q[i], c->h->q[i]);
        LAUNCH(c), k_prod_parts<G><<<dim3(gx1, 1, pg), 1024, smem, c->st>>>(last.p, pt, nullptr, l, nbp, c->pc, N, qi, c->dev_err);
        LimbMap lm{}; lm.n = 1; lm.prime[0] = (unsigned char)l;
        ntt_inplace(c, last.p, gnbp, lm, true);
        LAUNCH(c), k_centre_sum<<<dim3(c->gx(), gnbp), 256, 0, c->st>>>((i64 *)S.p, last.p, 1, gnbp, l, c->pc, N);
        LAUNCH(c), k_lift_mod<<<c->egrid(gnbp * l), 256, 0, c->st>>>(t.p, (const i64 *)S.p, l, c->pc, N);
        ntt_inplace(c, t.p, gnbp * l, c->qmap(l - 1), false);
        LAUNCH(c), k_prod_parts<G><<<dim3(gx1, (unsigned)l, pg), 1024, smem, c->st>>>(r->d, pt, t.p, l, nbp, c->pc, N, qi, c->dev_err);
        CK(cudaGetLastError());
    } catch (...) { hb_ct_free(r); throw; }
    return r;
}
template <int T>
void launch_matmul_tiles(hb_ctx *c, const hb_ct *pre, int btotal, int b0, const hb_pt *const *pts, int bcount, int kc, const u32 *dg, hb_ct *const *outs) {
    TilePts<T> tp{};
    for (int t = 0; t < T; ++t) {
        for (int b = 0; b < bcount; ++b) tp.p[t][b] = pts[(size_t)t * bcount + b]->d;
        tp.out[t] = outs[t]->d;
    }
    const int n = pre->level + 1;
    LAUNCH(c), k_matmul_acc_tiles<T><<<dim3((unsigned)(c->N / 512), (unsigned)(2 * n)), 256, 0, c->st>>>(tp, pre->d, kc, btotal, b0, bcount, dg, n, c->qmap(pre->level), c->pc, c->logn, c->N);
}
hb_ct *do_level_down(hb_ctx *c, const hb_ct *a, int target) {
    own(c, a);
    if (target > a->level || target < 0) fail(HB_E_LEVEL, "level_down: bad target");
    if (a->spow != 1) fail(HB_E_SHAPE, "level_down: operand not rescaled");
    const int N = c->N, nbp = a->batch * a->np, tl = target + 1;
    hb_ct *t = new_ct(c, tl, a->np, a->batch, 2);
    hb_ct *r = nullptr;
    try {
        const double cf = c->h->scale[target] * (double)c->h->q[tl] / c->h->scale[a->level];
        const i64 k = (i64)std::rint(cf);
        Scalars s{};
        for (int i = 0; i <= tl; ++i) s.v[i] = (u64)(k % (i64)c->h->q[i]);
        ALG(c, (size_t)nbp * (tl + 1)); // the input limbs that survive; do_rescale counts the rest
        LAUNCH(c), k_scalar_mul<<<c->egrid(nbp * (tl + 1)), 256, 0, c->st>>>(t->d, a->d, (size_t)(a->level + 1) * N, c->qmap(tl), c->pc, N, s);
        CK(cudaGetLastError());
        r = do_rescale(c, t);
    } catch (...) { hb_ct_free(t); throw; }
    hb_ct_free(t);
    return r;
}
hb_ct *do_addsub(hb_ctx *c, const hb_ct *a, const hb_ct *b, int mode) {
    own(c, a, b);
    if (a->level != b->level) { // level-adjusting add: bring the higher operand down first
        const hb_ct *hi = a->level > b->level ? a : b;
        hb_ct *low = do_level_down(c, hi, std::min(a->level, b->level));
        hb_ct *r = nullptr;
        try { r = hi == a ? do_addsub(c, low, b, mode) : do_addsub(c, a, low, mode); } catch (...) { hb_ct_free(low); throw; }
        hb_ct_free(low);
        return r;
    }
    check_same(a, b, "add");
    hb_ct *r = new_ct(c, a->level, a->np, a->batch, a->spow);
    ALG(c, 3 * a->limbs());
    LAUNCH(c), k_addsub<<<c->egrid((int)a->limbs()), 256, 0, c->st>>>(r->d, a->d, b->d, c->qmap(a->level), c->pc, c->N, mode);
    return r;
}
// acc (+)= sum over `groups` of tensor(a[g], b[g]); a, b hold groups * batch members, group-major
hb_ct *do_tensor(hb_ctx *c, const hb_ct *a, const hb_ct *b, hb_ct *acc, int groups = 1) {
    own(c, a, b, acc);
    check_same(a, b, "tensor");
    if (a->np != 2 || a->spow != 1) fail(HB_E_SHAPE, "tensor: operands must be rescaled 2-poly ciphertexts");
    if (groups < 1 || groups > kMaxRotGroups || a->batch % groups) fail(HB_E_SHAPE, "tensor: the batch does not split into that many groups");
    const int batch = a->batch / groups;
    hb_ct *r = acc;
    if (r) { if (r->level != a->level || r->np != 3 || r->batch != batch || r->spow != 2) fail(HB_E_SHAPE, "tensor_acc: accumulator mismatch"); }
    else r = new_ct(c, a->level, 3, batch, 2);
    const int n = a->level + 1;
    ALG(c, 2 * a->limbs() + (size_t)(acc ? 2 : 1) * batch * 3 * n);
    LAUNCH(c), k_tensor<<<c->egrid(batch * n), 256, 0, c->st>>>(r->d, a->d, b->d, n, c->qmap(a->level), c->pc, c->N, acc ? 1 : 0, groups, batch);
    return r;
}
hb_ct *do_relin(hb_ctx *c, const hb_ct *a) {
    own(c, a);
    if (a->np != 3) fail(HB_E_SHAPE, "relin: needs 3 polys");
    if (!c->mult_key.d) fail(HB_E_NOKEY, "multiplication key not generated");
    const int n = a->level + 1, N = c->N;
    hb_ct *r = new_ct(c, a->level, 2, a->batch, a->spow);
    ALG(c, (size_t)a->batch * 5 * n + key_limbs(c, a->level));
    try {
        keyswitch(c, a->d + (size_t)2 * n * N, (size_t)3 * n * N, a->level, a->batch, c->mult_key, 0, r->d, (size_t)2 * n * N, a->d, a->d + (size_t)n * N, (size_t)3 * n * N);
    } catch (...) { hb_ct_free(r); throw; }
    return r;
}
hb_ct *do_galois(hb_ctx *c, const hb_ct *a, u64 g) {
    own(c, a);
    if (a->np != 2) fail(HB_E_SHAPE, "rotate: needs 2 polys");
    const int n = a->level + 1, N = c->N;
    if (g == 1) { hb_ct *r = new_ct(c, a->level, 2, a->batch, a->spow); CK(cudaMemcpyAsync(r->d, a->d, a->limbs() * N * 8, cudaMemcpyDeviceToDevice, c->st)); return r; }
    const Evk &key = galois_key(c, g);
    hb_ct *r = new_ct(c, a->level, 2, a->batch, a->spow);
    ALG(c, (size_t)a->batch * 4 * n + key_limbs(c, a->level));
    try {
        keyswitch(c, a->d + (size_t)n * N, (size_t)2 * n * N, a->level, a->batch, key, (u32)g, r->d, (size_t)2 * n * N, a->d, nullptr, (size_t)2 * n * N);
    } catch (...) { hb_ct_free(r); throw; }
    return r;
}
hb_ct *do_mul_pt(hb_ctx *c, const hb_ct *a, const hb_pt *p) {
    own(c, a); own(c, p);
    if (a->level != p->level) fail(HB_E_LEVEL, "mul_pt: level mismatch");
    if (a->spow != 1 || p->spow != 1) fail(HB_E_SHAPE, "mul_pt: operand not rescaled");
    hb_ct *r = new_ct(c, a->level, a->np, a->batch, 2);
    ALG(c, 2 * a->limbs() + a->level + 1);
    LAUNCH(c), k_mul_pt<<<c->egrid((int)a->limbs()), 256, 0, c->st>>>(r->d, a->d, p->d, c->qmap(a->level), c->pc, c->N);
    return r;
}

// ---- allocation-free rescale ---------------------------------------------------------------
// Scratch for hb_rescale_noalloc lives in the library image instead of coming from cudaMalloc or the
// context's pool, so the call can be made by code that is not allowed to allocate device memory
// (for example a caller running under a fixed memory budget that was handed out in full at start-up,
// or one that must not disturb another allocator's view of the device).  Every GPU that loads the
// library holds these kNoAllocWords * 8 bytes (13 MiB) until the process exits.
constexpr size_t kNoAllocLimbs = 26;                      // one 2-poly ciphertext at level 12: 2 + 2*12 limbs
constexpr size_t kNoAllocWords = kNoAllocLimbs * 65536;   // of 2^16 words each
static __device__ __align__(256) unsigned long long g_noalloc_scratch[kNoAllocWords];
constexpr int kMaxDevices = 64;
u64 *g_noalloc_ptr[kMaxDevices] = {nullptr};

// Device address of the scratch array on the current device.  The array's name is only a host-side
// stand-in here; kernels must be given the address cudaGetSymbolAddress returns for this device.
u64 *noalloc_scratch(int device) {
    if (device < 0 || device >= kMaxDevices) fail(HB_E_LIMIT, "device index beyond the scratch table");
    if (!g_noalloc_ptr[device]) {
        void *p = nullptr;
        CK(cudaGetSymbolAddress(&p, g_noalloc_scratch));
        g_noalloc_ptr[device] = (u64 *)p;
    }
    return g_noalloc_ptr[device];
}

// host threads for the encode / decode halves of hb_encrypt_many / hb_decrypt_many
int host_workers(const hb_ctx *c, int tasks) {
    const int cap = c->host_threads > 0 ? c->host_threads : std::min(32, std::max(1, (int)std::thread::hardware_concurrency()));
    return std::max(1, std::min(tasks, cap));
}

template <class F> int guard(hb_ctx *c, F &&f) {
    try { CK(cudaSetDevice(c->device)); f(); return HB_OK; }
    catch (const ArgFail &e) { c->err = e.msg; return e.code; }
    catch (const CudaFail &e) { c->err = std::string(e.where) + ": " + cudaGetErrorString(e.e); return HB_E_CUDA; }
    catch (const std::invalid_argument &e) { c->err = e.what(); return HB_E_ARG; }
    catch (const std::exception &e) { c->err = e.what(); return HB_E_CUDA; }
}

} // namespace

extern "C" {

int hb_ctx_create(const hb_params *prm, int device, hb_ctx **out) {
    if (!prm || !out) return HB_E_ARG;
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || device < 0 || device >= ndev) { cudaGetLastError(); return HB_E_CUDA; }
    hb_ctx *c = new hb_ctx();
    try {
        HostParams hp{prm->log_n, prm->max_level, prm->dnum, prm->num_special, prm->q0_bits, prm->q_bits, prm->p_bits, prm->hamming_weight, prm->sigma,
                      {prm->seed[0], prm->seed[1], prm->seed[2], prm->seed[3]}};
        c->h.reset(new HostCtx(hp));
        if (!(c->h->logn == 16 || (c->h->logn >= 10 && c->h->logn <= 12))) throw std::invalid_argument("log_n must be 16, or 10..12 for small test contexts");
        if (c->h->digit_of(c->h->L) + 1 > 8) throw std::invalid_argument("more than 8 key-switch digits");
        c->device = device; c->N = c->h->N; c->logn = c->h->logn; c->L = c->h->L; c->K = c->h->K; c->nprimes = c->h->nprimes;
        for (int i = 0; i < 8; ++i) c->ckey.k[i] = c->h->cha.key[i];
        CK(cudaSetDevice(device));
        CK(cudaStreamCreateWithFlags(&c->st, cudaStreamNonBlocking));
        CK(cudaMalloc(&c->dev_err, sizeof(int)));
        CK(cudaMemset(c->dev_err, 0, sizeof(int)));
        const int np = c->nprimes, N = c->N;
        std::vector<PrimeConst> pcs(np);
        const bool big = c->logn == 16;   // 2^16 coefficients: tables in the order the two-pass kernels read them
        std::vector<u64> tw(big ? 0 : (size_t)4 * np * N);
        std::vector<ulonglong2> t16(big ? (size_t)2 * np * Ntt16Layout::kEntries : 0);
        std::vector<double> b8(big ? (size_t)2 * np * kRowsB8 : 0);
        for (int i = 0; i < np; ++i) {
            const u64 q = c->h->q[i];
            PrimeConst &p = pcs[i];
            p.q = q;
            unsigned __int128 two64 = (unsigned __int128)1 << 64;
            p.mu_hi = (u64)(two64 / q);
            p.mu_lo = (u64)(((two64 % q) << 64) / q);
            p.n_inv = hbhost::invmod((u64)N, q); p.n_inv_sh = hbhost::shoup(p.n_inv, q);
            p.iu = hbhost::powmod(c->h->psi_root[i], (u64)N / 2, q); p.iu_sh = hbhost::shoup(p.iu, q);
            // the 2^16 transform carries the residues of primes below 2^44 as integer-valued doubles (ntt16.cuh)
            p.small = (big && q < ((u64)1 << 44)) ? 1 : 0;
            p.q_inv_f = 1.0 / (double)q;
            p.n_inv_f = (double)p.n_inv / (double)q;
            p.fp = q < ((u64)1 << 44) ? 1 : 0;
            // lazy FP64-assisted products are below 1.6 q; reduce_fp takes sums below 2^52.  Every fixed-length lazy sum in
            // the kernels has at most 128 terms (16 rotated terms x 8 digits), which any prime below 2^44 allows (>= 160);
            // the open-ended sum of k_matmul_acc folds at this count.
            p.lazy_terms = (u64)((((unsigned __int128)1 << 52) * 5) / ((unsigned __int128)q * 8));
            if (p.fp && p.lazy_terms < 160) throw std::invalid_argument("prime too large for the lazy FP64-assisted sums");
            std::vector<u64> f, fs, iv, ivs;
            c->h->twiddles(i, f, fs, iv, ivs);
            if (p.small) { // companion words hold w/q as doubles instead of Shoup quotients
                for (int k = 0; k < N; ++k) {
                    double a = (double)f[k] / (double)q, b = (double)iv[k] / (double)q;
                    std::memcpy(&fs[k], &a, 8); std::memcpy(&ivs[k], &b, 8);
                }
            }
            if (big) {
                auto word = [&](u64 w) { return p.small ? ds_twiddle_word(w) : w; };
                ntt16_fill_table(&t16[(size_t)i * Ntt16Layout::kEntries], [&](unsigned k) { return make_ulonglong2(word(f[k]), fs[k]); });
                ntt16_fill_table(&t16[((size_t)np + i) * Ntt16Layout::kEntries], [&](unsigned k) { return make_ulonglong2(word(iv[k]), ivs[k]); });
                if (p.small) {
                    ntt16_fill_rows_b8(&b8[(size_t)i * kRowsB8], [&](unsigned k) { return (double)f[k]; });
                    ntt16_fill_rows_b8(&b8[((size_t)np + i) * kRowsB8], [&](unsigned k) { return (double)iv[k]; });
                }
            } else {
                std::memcpy(&tw[((size_t)0 * np + i) * N], f.data(), (size_t)N * 8);
                std::memcpy(&tw[((size_t)1 * np + i) * N], fs.data(), (size_t)N * 8);
                std::memcpy(&tw[((size_t)2 * np + i) * N], iv.data(), (size_t)N * 8);
                std::memcpy(&tw[((size_t)3 * np + i) * N], ivs.data(), (size_t)N * 8);
            }
        }
        CK(cudaMalloc(&c->pc, sizeof(PrimeConst) * np));
        CK(cudaMemcpy(c->pc, pcs.data(), sizeof(PrimeConst) * np, cudaMemcpyHostToDevice));
        if (big) {
            const size_t t16_bytes = t16.size() * sizeof(ulonglong2);
            CK(cudaMalloc(&c->tw, t16_bytes + b8.size() * sizeof(double)));
            CK(cudaMemcpy(c->tw, t16.data(), t16_bytes, cudaMemcpyHostToDevice));
            CK(cudaMemcpy(reinterpret_cast<char *>(c->tw) + t16_bytes, b8.data(), b8.size() * sizeof(double), cudaMemcpyHostToDevice));
            const ulonglong2 *t = reinterpret_cast<const ulonglong2 *>(c->tw);
            const double *tb8 = reinterpret_cast<const double *>(reinterpret_cast<const char *>(c->tw) + t16_bytes);
            c->tb.t16 = Ntt16Tables{t, t + (size_t)np * Ntt16Layout::kEntries, tb8, tb8 + (size_t)np * kRowsB8};
        } else {
            CK(cudaMalloc(&c->tw, tw.size() * 8));
            CK(cudaMemcpy(c->tw, tw.data(), tw.size() * 8, cudaMemcpyHostToDevice));
            c->tb.psi = c->tw; c->tb.psi_sh = c->tw + (size_t)np * N; c->tb.ipsi = c->tw + (size_t)2 * np * N; c->tb.ipsi_sh = c->tw + (size_t)3 * np * N;
        }
        CK(cudaMalloc(&c->sk, (size_t)np * N * 8));
    } catch (const CudaFail &) { hb_ctx_destroy(c); return HB_E_CUDA; }
    catch (const ArgFail &e) { int code = e.code; hb_ctx_destroy(c); return code; }
    catch (...) { hb_ctx_destroy(c); return HB_E_ARG; }
    *out = c;
    return HB_OK;
}
void hb_ctx_destroy(hb_ctx *c) {
    if (!c) return;
    cudaSetDevice(c->device);
    if (c->st) cudaStreamSynchronize(c->st);
    for (auto &kv : c->plans) cudaFree(kv.second);
    for (auto &kv : c->div_plans) cudaFree(kv.second);
    for (auto &kv : c->gal_tables) cudaFree(kv.second);
    if (c->pinned) cudaFreeHost(c->pinned);
    if (c->pc) cudaFree(c->pc);
    if (c->tw) cudaFree(c->tw);
    if (c->sk) cudaFree(c->sk);
    if (c->dev_err) cudaFree(c->dev_err);
    if (c->st) cudaStreamDestroy(c->st);
    delete c;
}
const char *hb_last_error(const hb_ctx *c) { return c ? c->err.c_str() : "null context"; }
int hb_ctx_info(const hb_ctx *c, uint64_t *primes, double *scales) {
    if (!c) return HB_E_ARG;
    if (primes) for (int i = 0; i < c->nprimes; ++i) primes[i] = c->h->q[i];
    if (scales) for (int i = 0; i <= c->L; ++i) scales[i] = c->h->scale[i];
    return HB_OK;
}
int hb_ctx_dims(const hb_ctx *c, int *log_n, int *max_level, int *num_special) {
    if (!c) return HB_E_ARG;
    if (log_n) *log_n = c->logn; if (max_level) *max_level = c->L; if (num_special) *num_special = c->K;
    return HB_OK;
}
int hb_sync(hb_ctx *c) {
    return guard(c, [&] {
        no_capture(c, "sync");
        int flag = 0;
        CK(cudaMemcpyAsync(&flag, c->dev_err, sizeof(int), cudaMemcpyDeviceToHost, c->st));
        CK(cudaStreamSynchronize(c->st));
        if (flag) {
            CK(cudaMemsetAsync(c->dev_err, 0, sizeof(int), c->st));
            fail(HB_E_TIMEOUT, "a bounded wait inside a kernel ran out; the results since the last sync are void");
        }
    });
}
int hb_mem_info(const hb_ctx *c, uint64_t *pool_bytes, uint64_t *in_use) {
    if (pool_bytes) *pool_bytes = c->pool.total;
    if (in_use) *in_use = c->pool.in_use;
    return HB_OK;
}
int hb_selftest_bounded_wait(hb_ctx *c) {
    return guard(c, [&] {
        no_capture(c, "selftest");
        LAUNCH(c), k_bounded_wait_probe<<<1, 32, 0, c->st>>>(c->dev_err, 64);
        CK(cudaGetLastError());
    });
}
int hb_release_cached(hb_ctx *c) {
    return guard(c, [&] {
        no_capture(c, "release_cached");
        CK(cudaStreamSynchronize(c->st));
        c->pool.release_cached();
    });
}
void *hb_stream(const hb_ctx *c) { return (void *)c->st; }
uint64_t hb_launch_count(const hb_ctx *c) { return c ? c->launches : 0; }
uint64_t hb_algorithmic_bytes(const hb_ctx *c) { return c ? c->alg_limbs * (uint64_t)c->N * 8 : 0; }

int hb_keygen(hb_ctx *c) {
    return guard(c, [&] {
        no_capture(c, "keygen");
        const HostCtx &h = *c->h;
        std::vector<i64> s; h.sample_secret(s);
        TmpBytes sc_buf(c, (size_t)c->N * 8);
        i64 *sc = (i64 *)sc_buf.p;
        CK(cudaMemcpyAsync(sc, s.data(), (size_t)c->N * 8, cudaMemcpyHostToDevice, c->st));
        const LimbMap am = c->allmap();
        LAUNCH(c), k_reduce_i64<<<c->egrid(c->nprimes), 256, 0, c->st>>>(c->sk, sc, am, c->pc, c->N);
        ntt_inplace(c, c->sk, c->nprimes, am, false);
        CK(cudaStreamSynchronize(c->st));
        c->have_sk = true;
        if (!c->mult_key.d) c->mult_key = make_key(c, 0, 0);
        const u64 gc = h.galois_conj();
        if (!c->gal_keys.count(gc)) c->gal_keys[gc] = make_key(c, gc, (u32)gc);
    });
}
int hb_gen_rot_keys(hb_ctx *c, const int64_t *steps, int n) {
    return guard(c, [&] {
        for (int i = 0; i < n; ++i) {
            const u64 g = c->h->galois_rot(steps[i]);
            if (g == 1 || c->gal_keys.count(g)) continue;
            c->gal_keys[g] = make_key(c, g, (u32)g);
        }
    });
}
uint64_t hb_galois_for_rotation(const hb_ctx *c, int64_t s) { return c->h->galois_rot(s); }
int hb_evk_export(hb_ctx *c, uint64_t g, uint64_t *host, int *digits) {
    return guard(c, [&] {
        no_capture(c, "evk_export");
        const Evk *k = g == 0 ? &c->mult_key : &galois_key(c, g);
        if (!k->d) fail(HB_E_NOKEY, "key not generated");
        if (digits) *digits = k->nd;
        if (host) { CK(cudaStreamSynchronize(c->st)); CK(cudaMemcpy(host, k->d, (size_t)k->nd * 2 * c->nprimes * c->N * 8, cudaMemcpyDeviceToHost)); }
    });
}

int hb_encode(hb_ctx *c, const double *re, const double *im, size_t n, int level, hb_pt **out) {
    return guard(c, [&] {
        no_capture(c, "encode");
        if (!re || !out || n > (size_t)c->h->slots) fail(HB_E_ARG, "encode: bad message");
        if (level < 0 || level > c->L) fail(HB_E_LEVEL, "encode: bad level");
        std::vector<i64> coef;
        c->h->encode_coeffs(re, im, n, c->h->scale[level], coef);
        hb_pt *p = new_pt(c, level, 1);
        try {
            TmpBytes dcb(c, (size_t)c->N * 8);
            i64 *dc = (i64 *)dcb.p;
            CK(cudaMemcpyAsync(dc, coef.data(), (size_t)c->N * 8, cudaMemcpyHostToDevice, c->st));
            const LimbMap qm = c->qmap(level);
            LAUNCH(c), k_reduce_i64<<<c->egrid(level + 1), 256, 0, c->st>>>(p->d, dc, qm, c->pc, c->N);
            ntt_inplace(c, p->d, level + 1, qm, false);
            CK(cudaStreamSynchronize(c->st)); // coef goes out of scope
        } catch (...) { hb_pt_free(p); throw; }
        *out = p;
    });
}
int hb_encode_ext(hb_ctx *c, const double *re, const double *im, size_t n, int level, hb_pt **out) {
    return guard(c, [&] {
        no_capture(c, "encode_ext");
        if (!re || !out || n > (size_t)c->h->slots) fail(HB_E_ARG, "encode: bad message");
        if (level < 0 || level > c->L) fail(HB_E_LEVEL, "encode: bad level");
        std::vector<i64> coef;
        c->h->encode_coeffs(re, im, n, c->h->scale[level], coef);
        const int ne = level + 1 + c->K;
        hb_pt *p = new hb_pt{c, level, 1, nullptr};
        p->ext = 1;
        try { p->d = c->alloc_limbs((size_t)ne); } catch (...) { delete p; throw; }
        try {
            TmpBytes dcb(c, (size_t)c->N * 8);
            i64 *dc = (i64 *)dcb.p;
            CK(cudaMemcpyAsync(dc, coef.data(), (size_t)c->N * 8, cudaMemcpyHostToDevice, c->st));
            LimbMap em{}; em.n = ne;
            for (int j = 0; j < ne; ++j) em.prime[j] = (unsigned char)(j <= level ? j : c->L + 1 + (j - level - 1));
            LAUNCH(c), k_reduce_i64<<<c->egrid(ne), 256, 0, c->st>>>(p->d, dc, em, c->pc, c->N);
            ntt_inplace(c, p->d, ne, em, false);
            CK(cudaStreamSynchronize(c->st)); // coef goes out of scope
        } catch (...) { hb_pt_free(p); throw; }
        *out = p;
    });
}
static void decode_limbs(hb_ctx *c, const u64 *dev_coef, int level, int spow, double *re, double *im) {
    const int nl = level >= 1 ? 2 : 1, N = c->N;
    std::vector<u64> hc((size_t)nl * N);
    CK(cudaMemcpyAsync(hc.data(), dev_coef, hc.size() * 8, cudaMemcpyDeviceToHost, c->st));
    CK(cudaStreamSynchronize(c->st));
    std::vector<double> val;
    c->h->centre(hc.data(), nl == 2 ? hc.data() + N : nullptr, val);
    const double sc = spow == 2 ? c->h->scale[level] * c->h->scale[level] : c->h->scale[level];
    c->h->decode_values(val, sc, re, im);
}
int hb_decode(hb_ctx *c, const hb_pt *p, double *re, double *im) {
    return guard(c, [&] {
        no_capture(c, "decode");
        const int nl = p->level >= 1 ? 2 : 1;
        Tmp t(c, (size_t)nl);
        ntt(c, p->d, (size_t)nl * c->N, t.p, (size_t)nl * c->N, nl, c->qmap(nl - 1), true);
        decode_limbs(c, t.p, p->level, p->spow, re, im);
    });
}
int hb_encrypt(hb_ctx *c, const hb_pt *p, uint64_t nonce, hb_ct **out) {
    return guard(c, [&] {
        no_capture(c, "encrypt");
        if (!c->have_sk) fail(HB_E_NOKEY, "secret key not generated");
        const int n = p->level + 1, N = c->N;
        hb_ct *r = new_ct(c, p->level, 2, 1, p->spow);
        try {
            const LimbMap qm = c->qmap(p->level);
            u64 *b = r->d, *a = r->d + (size_t)n * N;
            LAUNCH(c), k_uniform<<<dim3((unsigned)((N / 4 + 255) / 256), n), 256, 0, c->st>>>(a, qm, c->pc, N, c->ckey, hbhost::STREAM_ENC_A, nonce);
            std::vector<i64> ev; c->h->sample_gauss(hbhost::STREAM_ENC_E, nonce, ev);
            TmpBytes ecb(c, (size_t)N * 8);
            i64 *ec = (i64 *)ecb.p;
            Tmp e(c, (size_t)n);
            CK(cudaMemcpyAsync(ec, ev.data(), (size_t)N * 8, cudaMemcpyHostToDevice, c->st));
            LAUNCH(c), k_reduce_i64<<<c->egrid(n), 256, 0, c->st>>>(e.p, ec, qm, c->pc, N);
            ntt_inplace(c, e.p, n, qm, false);
            LAUNCH(c), k_encrypt<<<c->egrid(n), 256, 0, c->st>>>(b, a, e.p, c->sk, p->d, qm, c->pc, N);
            CK(cudaStreamSynchronize(c->st));
        } catch (...) { hb_ct_free(r); throw; }
        *out = r;
    });
}
// encode + encrypt `count` messages into one batched handle; member i is bit for bit hb_encrypt(hb_encode(message i), nonces[i])
int hb_encrypt_many(hb_ctx *c, const double *re, const double *im, size_t n_slots, int count, int level, const uint64_t *nonces, hb_ct **out) {
    return guard(c, [&] {
        no_capture(c, "encrypt_many");
        if (!c->have_sk) fail(HB_E_NOKEY, "secret key not generated");
        if (!re || !nonces || !out || count < 1 || n_slots > (size_t)c->h->slots) fail(HB_E_ARG, "encrypt_many: bad message");
        if (level < 0 || level > c->L) fail(HB_E_LEVEL, "encrypt_many: bad level");
        const int n = level + 1, N = c->N;
        const HostCtx &h = *c->h;
        // host part, one member per task: inverse embedding + rounding, and the error polynomial
        const size_t words = (size_t)count * 2 * N;
        if (c->pinned_bytes < words * 8) {
            if (c->pinned) CK(cudaFreeHost(c->pinned));
            c->pinned = nullptr; c->pinned_bytes = 0;
            CK(cudaMallocHost(&c->pinned, words * 8));
            c->pinned_bytes = words * 8;
        }
        i64 *host = (i64 *)c->pinned; // [count][2][N]: message coefficients, error coefficients
        const int workers = host_workers(c, count);
        std::vector<std::thread> pool;
        for (int w = 0; w < workers; ++w)
            pool.emplace_back([&, w] {
                std::vector<i64> v;
                for (int i = w; i < count; i += workers) {
                    h.encode_coeffs(re + (size_t)i * n_slots, im ? im + (size_t)i * n_slots : nullptr, n_slots, h.scale[level], v);
                    std::memcpy(host + (size_t)i * 2 * N, v.data(), (size_t)N * 8);
                    h.sample_gauss(hbhost::STREAM_ENC_E, nonces[i], v);
                    std::memcpy(host + ((size_t)i * 2 + 1) * N, v.data(), (size_t)N * 8);
                }
            });
        for (auto &th : pool) th.join();
        hb_ct *r = new_ct(c, level, 2, count, 1);
        try {
            const LimbMap qm = c->qmap(level);
            TmpBytes dcb(c, words * 8);
            i64 *dc = (i64 *)dcb.p;
            Tmp me(c, (size_t)count * 2 * n); // [count][message | error][n][N]
            CK(cudaMemcpyAsync(dc, host, words * 8, cudaMemcpyHostToDevice, c->st));
            for (int i = 0; i < count * 2; ++i)
                LAUNCH(c), k_reduce_i64<<<c->egrid(n), 256, 0, c->st>>>(me.p + (size_t)i * n * N, dc + (size_t)i * N, qm, c->pc, N);
            ntt_inplace(c, me.p, count * 2 * n, qm, false);
            for (int i = 0; i < count; ++i) {
                u64 *b = r->d + (size_t)i * 2 * n * N, *a = b + (size_t)n * N;
                LAUNCH(c), k_uniform<<<dim3((unsigned)((N / 4 + 255) / 256), n), 256, 0, c->st>>>(a, qm, c->pc, N, c->ckey, hbhost::STREAM_ENC_A, nonces[i]);
                LAUNCH(c), k_encrypt<<<c->egrid(n), 256, 0, c->st>>>(b, a, me.p + ((size_t)i * 2 + 1) * n * N, c->sk, me.p + (size_t)i * 2 * n * N, qm, c->pc, N);
            }
            CK(cudaGetLastError());
            CK(cudaStreamSynchronize(c->st)); // the staging buffer is reused by the next call
        } catch (...) { hb_ct_free(r); throw; }
        *out = r;
    });
}
int hb_decrypt(hb_ctx *c, const hb_ct *ct, int index, double *re, double *im) {
    return guard(c, [&] {
        no_capture(c, "decrypt");
        if (!c->have_sk) fail(HB_E_NOKEY, "secret key not generated");
        if (index < 0 || index >= ct->batch) fail(HB_E_ARG, "decrypt: bad batch index");
        const int n = ct->level + 1, N = c->N, nl = ct->level >= 1 ? 2 : 1;
        Tmp t(c, (size_t)nl);
        LAUNCH(c), k_decrypt<<<c->egrid(nl), 256, 0, c->st>>>(t.p, ct->d + (size_t)index * ct->np * n * N, n, ct->np, c->sk, c->pc, N);
        ntt_inplace(c, t.p, nl, c->qmap(nl - 1), true);
        decode_limbs(c, t.p, ct->level, ct->spow, re, im);
    });
}

int hb_decrypt_many(hb_ctx *c, const hb_ct *const *cts, const int *index, int count, double *re, double *im) {
    return guard(c, [&] {
        no_capture(c, "decrypt_many");
        if (!c->have_sk) fail(HB_E_NOKEY, "secret key not generated");
        if (count < 1 || !cts || !re) fail(HB_E_ARG, "decrypt_many: nothing to decrypt");
        const int N = c->N, slots = c->h->slots;
        bool two = true;
        for (int i = 0; i < count; ++i) {
            const int idx = index ? index[i] : 0;
            if (!cts[i] || idx < 0 || idx >= cts[i]->batch) fail(HB_E_ARG, "decrypt_many: bad batch index");
            if (cts[i]->level < 1) two = false;
        }
        if (!two) { // a level-0 member has one limb only: take the members one by one
            for (int i = 0; i < count; ++i) {
                const hb_ct *ct = cts[i];
                const int n = ct->level + 1, nl = ct->level >= 1 ? 2 : 1;
                Tmp t(c, (size_t)nl);
                LAUNCH(c), k_decrypt<<<c->egrid(nl), 256, 0, c->st>>>(t.p, ct->d + (size_t)(index ? index[i] : 0) * ct->np * n * N, n, ct->np, c->sk, c->pc, N);
                ntt_inplace(c, t.p, nl, c->qmap(nl - 1), true);
                decode_limbs(c, t.p, ct->level, ct->spow, re + (size_t)i * slots, im ? im + (size_t)i * slots : nullptr);
            }
            return;
        }
        const size_t bytes = (size_t)count * 2 * N * 8;
        if (c->pinned_bytes < bytes) {
            if (c->pinned) CK(cudaFreeHost(c->pinned));
            c->pinned = nullptr; c->pinned_bytes = 0;
            CK(cudaMallocHost(&c->pinned, bytes));
            c->pinned_bytes = bytes;
        }
        Tmp t(c, (size_t)count * 2);
        for (int i = 0; i < count; ++i) {
            const hb_ct *ct = cts[i];
            const int n = ct->level + 1;
            LAUNCH(c), k_decrypt<<<c->egrid(2), 256, 0, c->st>>>(t.p + (size_t)i * 2 * N, ct->d + (size_t)(index ? index[i] : 0) * ct->np * n * N, n, ct->np, c->sk, c->pc, N);
        }
        ntt_inplace(c, t.p, count * 2, c->qmap(1), true);
        CK(cudaMemcpyAsync(c->pinned, t.p, bytes, cudaMemcpyDeviceToHost, c->st));
        CK(cudaStreamSynchronize(c->st));
        // CRT lift and inverse embedding on the host cores, one member per task
        const int workers = host_workers(c, count);
        std::vector<std::thread> pool;
        const HostCtx &h = *c->h;
        const u64 *host = c->pinned;
        for (int w = 0; w < workers; ++w)
            pool.emplace_back([&, w] {
                std::vector<double> val;
                for (int i = w; i < count; i += workers) {
                    const hb_ct *ct = cts[i];
                    h.centre(host + (size_t)i * 2 * N, host + ((size_t)i * 2 + 1) * N, val);
                    const double sc = ct->spow == 2 ? h.scale[ct->level] * h.scale[ct->level] : h.scale[ct->level];
                    h.decode_values(val, sc, re + (size_t)i * slots, im ? im + (size_t)i * slots : nullptr);
                }
            });
        for (auto &th : pool) th.join();
    });
}

int hb_ct_create(hb_ctx *c, int level, int np, int batch, int spow, hb_ct **out) { return guard(c, [&] { *out = new_ct(c, level, np, batch, spow); }); }
int hb_ct_clone(hb_ctx *c, const hb_ct *s, hb_ct **out) {
    return guard(c, [&] {
        hb_ct *r = new_ct(c, s->level, s->np, s->batch, s->spow);
        CK(cudaMemcpyAsync(r->d, s->d, s->limbs() * c->N * 8, cudaMemcpyDeviceToDevice, c->st));
        *out = r;
    });
}
int hb_ct_zero(hb_ctx *c, hb_ct *x) { return guard(c, [&] { own(c, x); CK(cudaMemsetAsync(x->d, 0, x->limbs() * c->N * 8, c->st)); }); }
void hb_ct_free(hb_ct *x) { if (x) { x->ctx->pool.put(x->d); delete x; } }
void hb_pt_free(hb_pt *x) { if (x) { x->ctx->pool.put(x->d); delete x; } }
int hb_ct_meta(const hb_ct *x, int *level, int *np, int *batch, int *spow) {
    if (!x) return HB_E_ARG;
    if (level) *level = x->level; if (np) *np = x->np; if (batch) *batch = x->batch; if (spow) *spow = x->spow;
    return HB_OK;
}
int hb_pt_meta(const hb_pt *x, int *level, int *spow) { if (!x) return HB_E_ARG; if (level) *level = x->level; if (spow) *spow = x->spow; return HB_OK; }
int hb_ct_import(hb_ctx *c, hb_ct *x, const uint64_t *host) {
    return guard(c, [&] { no_capture(c, "ct_import"); own(c, x); CK(cudaMemcpyAsync(x->d, host, x->limbs() * c->N * 8, cudaMemcpyHostToDevice, c->st)); CK(cudaStreamSynchronize(c->st)); });
}
int hb_ct_export(hb_ctx *c, const hb_ct *x, uint64_t *host) {
    return guard(c, [&] { no_capture(c, "ct_export"); own(c, x); CK(cudaMemcpyAsync(host, x->d, x->limbs() * c->N * 8, cudaMemcpyDeviceToHost, c->st)); CK(cudaStreamSynchronize(c->st)); });
}
int hb_pt_export(hb_ctx *c, const hb_pt *x, uint64_t *host) {
    return guard(c, [&] { no_capture(c, "pt_export"); own(c, x); CK(cudaMemcpyAsync(host, x->d, (size_t)(x->level + 1) * c->N * 8, cudaMemcpyDeviceToHost, c->st)); CK(cudaStreamSynchronize(c->st)); });
}
void *hb_ct_device_ptr(const hb_ct *x) { return x ? x->d : nullptr; }
int hb_batch_set(hb_ctx *c, hb_ct *dst, int idx, const hb_ct *src) {
    return guard(c, [&] {
        own(c, dst, src);
        if (src->level != dst->level || src->np != dst->np || idx < 0 || (idx + 1) * src->batch > dst->batch) fail(HB_E_SHAPE, "batch_set: mismatch");
        const size_t per = (size_t)src->batch * src->np * (src->level + 1) * c->N; // position counted in units of src's batch
        CK(cudaMemcpyAsync(dst->d + per * idx, src->d, per * 8, cudaMemcpyDeviceToDevice, c->st));
    });
}
int hb_batch_get(hb_ctx *c, const hb_ct *src, int idx, hb_ct **out) {
    return guard(c, [&] {
        if (idx < 0 || idx >= src->batch) fail(HB_E_ARG, "batch_get: bad index");
        hb_ct *r = new_ct(c, src->level, src->np, 1, src->spow);
        const size_t per = (size_t)src->np * (src->level + 1) * c->N;
        CK(cudaMemcpyAsync(r->d, src->d + per * idx, per * 8, cudaMemcpyDeviceToDevice, c->st));
        *out = r;
    });
}

int hb_batch_concat(hb_ctx *c, const hb_ct *const *parts, int n, hb_ct **out) {
    return guard(c, [&] {
        if (n < 1) fail(HB_E_ARG, "batch_concat: nothing to join");
        int total = 0;
        for (int k = 0; k < n; ++k) {
            if (parts[k]->level != parts[0]->level || parts[k]->np != parts[0]->np || parts[k]->spow != parts[0]->spow) fail(HB_E_SHAPE, "batch_concat: mismatch");
            total += parts[k]->batch;
        }
        hb_ct *r = new_ct(c, parts[0]->level, parts[0]->np, total, parts[0]->spow);
        size_t off = 0;
        for (int k = 0; k < n; ++k) {
            const size_t words = parts[k]->limbs() * c->N;
            CK(cudaMemcpyAsync(r->d + off, parts[k]->d, words * 8, cudaMemcpyDeviceToDevice, c->st));
            off += words;
        }
        *out = r;
    });
}
int hb_batch_slice(hb_ctx *c, const hb_ct *src, int start, int count, hb_ct **out) {
    return guard(c, [&] {
        if (start < 0 || count < 1 || start + count > src->batch) fail(HB_E_ARG, "batch_slice: bad range");
        hb_ct *r = new_ct(c, src->level, src->np, count, src->spow);
        const size_t per = (size_t)src->np * (src->level + 1) * c->N;
        CK(cudaMemcpyAsync(r->d, src->d + per * start, per * count * 8, cudaMemcpyDeviceToDevice, c->st));
        *out = r;
    });
}
int hb_add(hb_ctx *c, const hb_ct *a, const hb_ct *b, hb_ct **out) { return guard(c, [&] { *out = do_addsub(c, a, b, 0); }); }
int hb_sub(hb_ctx *c, const hb_ct *a, const hb_ct *b, hb_ct **out) { return guard(c, [&] { *out = do_addsub(c, a, b, 1); }); }
int hb_negate(hb_ctx *c, const hb_ct *a, hb_ct **out) {
    return guard(c, [&] {
        hb_ct *r = new_ct(c, a->level, a->np, a->batch, a->spow);
        ALG(c, 2 * a->limbs());
        LAUNCH(c), k_addsub<<<c->egrid((int)a->limbs()), 256, 0, c->st>>>(r->d, a->d, a->d, c->qmap(a->level), c->pc, c->N, 2);
        *out = r;
    });
}
int hb_mult_imag(hb_ctx *c, const hb_ct *a, hb_ct **out) {
    return guard(c, [&] {
        hb_ct *r = new_ct(c, a->level, a->np, a->batch, a->spow);
        ALG(c, 2 * a->limbs());
        LAUNCH(c), k_mult_imag<<<c->egrid((int)a->limbs()), 256, 0, c->st>>>(r->d, a->d, c->qmap(a->level), c->pc, c->N);
        *out = r;
    });
}
int hb_mult_int(hb_ctx *c, const hb_ct *a, int64_t k, hb_ct **out) {
    return guard(c, [&] {
        hb_ct *r = new_ct(c, a->level, a->np, a->batch, a->spow);
        Scalars s{};
        for (int i = 0; i <= a->level; ++i) { const i64 q = (i64)c->h->q[i]; i64 v = k % q; if (v < 0) v += q; s.v[i] = (u64)v; }
        ALG(c, 2 * a->limbs());
        LAUNCH(c), k_scalar_mul<<<c->egrid((int)a->limbs()), 256, 0, c->st>>>(r->d, a->d, (size_t)(a->level + 1) * c->N, c->qmap(a->level), c->pc, c->N, s);
        *out = r;
    });
}
int hb_mul_pt_norescale(hb_ctx *c, const hb_ct *a, const hb_pt *p, hb_ct **out) { return guard(c, [&] { *out = do_mul_pt(c, a, p); }); }
int hb_mul_pt(hb_ctx *c, const hb_ct *a, const hb_pt *p, hb_ct **out) { return guard(c, [&] { *out = do_prod_rescale(c, &a, &p, 1, true); }); }
int hb_mul_pt_sum(hb_ctx *c, const hb_ct *const *a, const hb_pt *const *p, int count, hb_ct **out) {
    return guard(c, [&] { *out = do_prod_rescale(c, a, p, count, true); });
}
int hb_sum_mul_pt_rescale(hb_ctx *c, const hb_ct *const *a, const hb_pt *const *p, int count, hb_ct **out) {
    return guard(c, [&] { *out = do_prod_rescale(c, a, p, count, false); });
}
int hb_rescale(hb_ctx *c, const hb_ct *a, hb_ct **out) { return guard(c, [&] { *out = do_rescale(c, a); }); }
int hb_rescale_noalloc(hb_ctx *c, const hb_ct *a, hb_ct *out) {
    return guard(c, [&] {
        if (!a || !out) fail(HB_E_ARG, "rescale_noalloc: null handle");
        own(c, a, out);
        if (a->level < 1) fail(HB_E_LEVEL, "rescale: level 0");
        if (a->spow != 2) fail(HB_E_SHAPE, "rescale: nothing to rescale");
        if (out->level != a->level - 1 || out->np != a->np || out->batch != a->batch) fail(HB_E_SHAPE, "rescale_noalloc: output handle must be level-1 with the same polys and batch");
        const int l = a->level, N = c->N, nbp = a->batch * a->np;
        const size_t need = (size_t)nbp * (1 + (size_t)l) * N;
        if (need > kNoAllocWords)
            fail(HB_E_LIMIT, "rescale_noalloc: needs " + std::to_string(need * 8) + " bytes of scratch, the built-in buffer holds " + std::to_string(kNoAllocWords * 8) +
                                 " (one 2-poly ciphertext at level 12 and N = 2^16)");
        u64 *scratch = noalloc_scratch(c->device); // first call on a device resolves the address
        u64 *last = scratch, *t = scratch + (size_t)nbp * N;
        LimbMap lm{}; lm.n = 1; lm.prime[0] = (unsigned char)l;
        ntt(c, a->d + (size_t)l * N, (size_t)(l + 1) * N, last, (size_t)N, nbp, lm, true);
        LAUNCH(c), k_rescale_prep<<<c->egrid(nbp * l), 256, 0, c->st>>>(t, last, l, c->pc, N);
        ntt_inplace(c, t, nbp * l, c->qmap(l - 1), false);
        Scalars qi{};
        for (int i = 0; i < l; ++i) qi.v[i] = hbhost::invmod(c->h->q[l] % c->h->q[i], c->h->q[i]);
        LAUNCH(c), k_rescale_fin<<<c->egrid(nbp * l), 256, 0, c->st>>>(out->d, a->d, t, l, c->pc, N, qi);
        CK(cudaGetLastError());
        out->spow = 1;
    });
}
int hb_level_down(hb_ctx *c, const hb_ct *a, int target, hb_ct **out) {
    return guard(c, [&] {
        if (target == a->level) { hb_ct *r = new_ct(c, a->level, a->np, a->batch, a->spow); CK(cudaMemcpyAsync(r->d, a->d, a->limbs() * c->N * 8, cudaMemcpyDeviceToDevice, c->st)); *out = r; }
        else *out = do_level_down(c, a, target);
    });
}
int hb_tensor(hb_ctx *c, const hb_ct *a, const hb_ct *b, hb_ct **out) { return guard(c, [&] { *out = do_tensor(c, a, b, nullptr); }); }
int hb_tensor_acc(hb_ctx *c, const hb_ct *a, const hb_ct *b, hb_ct **acc) { return guard(c, [&] { *acc = do_tensor(c, a, b, *acc); }); }
int hb_relin(hb_ctx *c, const hb_ct *a, hb_ct **out) { return guard(c, [&] { *out = do_relin(c, a); }); }
int hb_mul(hb_ctx *c, const hb_ct *a, const hb_ct *b, hb_ct **out) {
    return guard(c, [&] {
        if (a->level != b->level) { // align levels: the higher operand comes down first
            const hb_ct *hi = a->level > b->level ? a : b;
            hb_ct *low = do_level_down(c, hi, std::min(a->level, b->level));
            int rc = hi == a ? hb_mul(c, low, b, out) : hb_mul(c, a, low, out);
            hb_ct_free(low);
            if (rc != HB_OK) throw ArgFail{rc, c->err};
            return;
        }
        hb_ct *t = do_tensor(c, a, b, nullptr), *r = nullptr;
        try { r = do_relin(c, t); } catch (...) { hb_ct_free(t); throw; }
        hb_ct_free(t);
        try { *out = do_rescale(c, r); } catch (...) { hb_ct_free(r); throw; }
        hb_ct_free(r);
    });
}
// HomEvaluator::square (HomEvaluator.hpp:363): mult(a, a)
int hb_square(hb_ctx *c, const hb_ct *a, hb_ct **out) { return hb_mul(c, a, a, out); }
// HomEvaluator::mult(ct, Complex / Real constant) (HomEvaluator.hpp:275-278): the constant in every slot, encoded at the
// ciphertext's level, one rescale
int hb_mul_const(hb_ctx *c, const hb_ct *a, double re, double im, hb_ct **out) {
    if (!c || !a || !out) return HB_E_ARG;
    std::vector<double> vr((size_t)c->h->slots, re), vi((size_t)c->h->slots, im);
    hb_pt *p = nullptr;
    int rc = hb_encode(c, vr.data(), vi.data(), vr.size(), a->level, &p);
    if (rc != HB_OK) return rc;
    rc = hb_mul_pt(c, a, p, out);
    hb_pt_free(p);
    return rc;
}
int hb_decompose(hb_ctx *c, const hb_ct *a, hb_digits **out) {
    return guard(c, [&] {
        if (a->np != 2) fail(HB_E_SHAPE, "decompose: needs 2 polys");
        own(c, a);
        const PlanDims d = plan_dims(c, a->level);
        const int n = a->level + 1, N = c->N;
        hb_digits *h = new hb_digits{c, a->level, a->batch, nullptr};
        try {
            h->d = c->alloc_limbs((size_t)a->batch * d.dt_count);
            ALG(c, (size_t)a->batch * (n + d.dt_count));
            ks_decompose(c, a->d + (size_t)n * N, (size_t)2 * n * N, a->level, a->batch, h->d);
        } catch (...) { c->pool.put(h->d); delete h; throw; }
        *out = h;
    });
}
void hb_digits_free(hb_digits *h) { if (h) { h->ctx->pool.put(h->d); delete h; } }
int hb_rotate_hoisted(hb_ctx *c, const hb_ct *a, const hb_digits *dg, int64_t steps, hb_ct **out) {
    return guard(c, [&] {
        if (a->np != 2 || dg->level != a->level || dg->batch != a->batch) fail(HB_E_SHAPE, "rotate_hoisted: digits do not belong to this ciphertext");
        own(c, a); own(c, dg);
        const u64 g = c->h->galois_rot(steps);
        const int n = a->level + 1, N = c->N;
        hb_ct *r = new_ct(c, a->level, 2, a->batch, a->spow);
        if (g == 1) { CK(cudaMemcpyAsync(r->d, a->d, a->limbs() * N * 8, cudaMemcpyDeviceToDevice, c->st)); *out = r; return; }
        try {
            const Evk &key = galois_key(c, g);
            ALG(c, (size_t)a->batch * (4 * n + plan_dims(c, a->level).dt_count) + key_limbs(c, a->level));
            ks_apply(c, a->d + (size_t)n * N, (size_t)2 * n * N, dg->d, a->level, a->batch, key, (u32)g, r->d, (size_t)2 * n * N, a->d, nullptr, (size_t)2 * n * N);
        } catch (...) { hb_ct_free(r); throw; }
        *out = r;
    });
}
int hb_assemble_hoisted(hb_ctx *c, const hb_ct *a, const hb_digits *dg, int64_t s1, const hb_pt *p1, int64_t s2, const hb_pt *p2, hb_ct **out) {
    return guard(c, [&] {
        if (a->np != 2 || dg->level != a->level || dg->batch != a->batch) fail(HB_E_SHAPE, "assemble_hoisted: digits do not belong to this ciphertext");
        *out = do_assemble_rot(c, a, dg->d, s1, p1, s2, p2);
    });
}
int hb_assemble_rot(hb_ctx *c, const hb_ct *a, int64_t s1, const hb_pt *p1, int64_t s2, const hb_pt *p2, hb_ct **out) {
    return guard(c, [&] {
        if (a->np != 2) fail(HB_E_SHAPE, "assemble_rot: needs 2 polys");
        const PlanDims d = plan_dims(c, a->level);
        const int n = a->level + 1, N = c->N;
        Tmp dt(c, (size_t)a->batch * d.dt_count);
        ks_decompose(c, a->d + (size_t)n * N, (size_t)2 * n * N, a->level, a->batch, dt.p);
        *out = do_assemble_rot(c, a, dt.p, s1, p1, s2, p2);
    });
}
int hb_masked_key_create(hb_ctx *c, int64_t steps, const hb_pt *m1, const hb_pt *m2, hb_mkey **out) {
    return guard(c, [&] {
        if (!m1 || !m1->ext || m1->spow != 1 || (m2 && (!m2->ext || m2->level != m1->level || m2->spow != 1))) fail(HB_E_ARG, "masked_key: extended plaintexts of one level needed");
        const u64 g = c->h->galois_rot(steps);
        if (g == 1) fail(HB_E_ARG, "masked_key: zero rotation");
        const int level = m1->level, N = c->N;
        if (level < 1) fail(HB_E_LEVEL, "masked_key: level 0");
        const Evk &key = galois_key(c, g);
        const KsPlan *pl = get_plan(c, level);
        const DivPlan *dv = get_div_plan(c, level);
        const PlanDims d = plan_dims(c, level);
        hb_mkey *k = new hb_mkey{c, level, (u32)g, nullptr, nullptr};
        try {
            k->key = c->alloc_limbs((size_t)d.nd * 2 * d.ne);
            k->pm = c->alloc_limbs((size_t)d.n);
            LAUNCH(c), k_mask_key<<<dim3(c->gx(), d.ne, d.nd * 2), 256, 0, c->st>>>(k->key, key.d, c->nprimes, m1->d, m2 ? m2->d : nullptr, pl, c->pc, N);
            LAUNCH(c), k_mask_p<<<dim3(c->gx(), d.n), 256, 0, c->st>>>(k->pm, m1->d, m2 ? m2->d : nullptr, dv, c->pc, N);
            CK(cudaGetLastError());
        } catch (...) { if (k->key) c->pool.put(k->key); if (k->pm) c->pool.put(k->pm); delete k; throw; }
        *out = k;
    });
}
void hb_masked_key_free(hb_mkey *k) { if (k) { k->ctx->pool.put(k->key); k->ctx->pool.put(k->pm); delete k; } }
int hb_assemble_masked(hb_ctx *c, const hb_ct *a, const hb_digits *dg, const hb_mkey *k1, const hb_mkey *k2, hb_ct **out) {
    return guard(c, [&] {
        if (a->np != 2 || dg->level != a->level || dg->batch != a->batch) fail(HB_E_SHAPE, "assemble_masked: digits do not belong to this ciphertext");
        *out = do_assemble_mk(c, a, dg->d, &k1, k2 ? &k2 : nullptr, 1);
    });
}
int hb_assemble_masked_multi(hb_ctx *c, const hb_ct *a, const hb_digits *dg, const hb_mkey *const *k1s, const hb_mkey *const *k2s, int groups, hb_ct **out) {
    return guard(c, [&] {
        if (a->np != 2 || dg->level != a->level || dg->batch != a->batch) fail(HB_E_SHAPE, "assemble_masked: digits do not belong to this ciphertext");
        if (!k1s) fail(HB_E_ARG, "assemble_masked: no keys");
        *out = do_assemble_mk(c, a, dg->d, k1s, k2s, groups);
    });
}
int hb_tensor_acc_groups(hb_ctx *c, const hb_ct *a, const hb_ct *b, int groups, hb_ct **acc) { return guard(c, [&] { *acc = do_tensor(c, a, b, *acc, groups); }); }
// sum_t rot(xs[t], steps[t]): every term is decomposed, the inner products of all terms are added up in Q_level u P by
// one kernel, and one ModDown serves the sum; unrotated terms (step 0) are added as they are.
// sum_t rot(x_t, steps[t]) with one ModDown; x_t = `batch` members starting at base[t] (all of one shape)
static hb_ct *rotate_sum_core(hb_ctx *c, const u64 *const *base, const int64_t *steps, int count, int level, int batch, int spow, const u64 *dt_all, size_t dt_term_stride) {
    const int N = c->N;
    const KsPlan *pl = get_plan(c, level);
    const PlanDims d = plan_dims(c, level);
    const int n = d.n, ne = d.ne, K = d.K;
    const size_t ct_outer = (size_t)2 * n * N;
    RotTermList rot{}; PlainTermList plain{};
    std::vector<u64 *> dts;
    hb_ct *r = new_ct(c, level, 2, batch, spow);
    try {
        for (int t = 0; t < count; ++t) {
            const u64 g = c->h->galois_rot(steps[t]);
            if (g == 1) {
                if (plain.count == 16) fail(HB_E_LIMIT, "rotate_sum: at most 16 unrotated terms");
                plain.x[plain.count++] = base[t];
                continue;
            }
            if (rot.count == 16) fail(HB_E_LIMIT, "rotate_sum: at most 16 rotated terms");
            const Evk &key = galois_key(c, g);
            const u64 *dt;
            if (dt_all) dt = dt_all + (size_t)t * dt_term_stride;
            else {
                u64 *fresh = c->alloc_limbs((size_t)batch * d.dt_count);
                dts.push_back(fresh);
                ks_decompose(c, base[t] + (size_t)n * N, ct_outer, level, batch, fresh);
                dt = fresh;
            }
            rot.t[rot.count++] = RotTerm{base[t] + (size_t)n * N, dt, key.d, (u32)g, 0u};
        }
        const unsigned gx = c->gx();
        ALG(c, (size_t)(count + 1) * batch * 2 * n + (size_t)rot.count * key_limbs(c, level));
        Tmp add(c, (size_t)batch * 2 * n);
        LAUNCH(c), k_rot_sum_addend<<<dim3(gx, n, batch * 2), 256, 0, c->st>>>(add.p, rot, plain, n, c->qmap(level), c->pc, c->logn, N);
        if (rot.count == 0) {
            CK(cudaMemcpyAsync(r->d, add.p, r->limbs() * N * 8, cudaMemcpyDeviceToDevice, c->st));
        } else {
            Tmp acc(c, (size_t)batch * 2 * ne), pco(c, (size_t)batch * 2 * K), t(c, (size_t)batch * 2 * n);
            LAUNCH(c), k_ks_inner_sum<<<dim3(gx, batch, ne), 256, 0, c->st>>>(acc.p, rot, ct_outer, c->nprimes, pl, c->pc, c->logn, N);
            moddown(c, acc.p, pco.p, t.p, level, batch, r->d, ct_outer, add.p, add.p + (size_t)n * N, ct_outer, 0u);
        }
        CK(cudaGetLastError());
    } catch (...) { for (u64 *p : dts) c->pool.put(p); hb_ct_free(r); throw; }
    for (u64 *p : dts) c->pool.put(p);
    return r;
}
int hb_rotate_sum(hb_ctx *c, const hb_ct *const *xs, const int64_t *steps, int count, hb_ct **out) {
    return guard(c, [&] {
        if (count < 1 || count > 32 || !xs || !steps) fail(HB_E_LIMIT, "rotate_sum: 1 to 32 terms");
        const hb_ct *x0 = xs[0];
        for (int t = 0; t < count; ++t)
            if (!xs[t] || xs[t]->np != 2 || xs[t]->level != x0->level || xs[t]->batch != x0->batch || xs[t]->spow != x0->spow) fail(HB_E_SHAPE, "rotate_sum: operands differ in shape");
        std::vector<const u64 *> base((size_t)count);
        for (int t = 0; t < count; ++t) { own(c, xs[t]); base[(size_t)t] = xs[t]->d; }
        *out = rotate_sum_core(c, base.data(), steps, count, x0->level, x0->batch, x0->spow, nullptr, 0);
    });
}
// the same when the terms are the member groups of one ciphertext (group t = members t * batch/groups ...): the digits of
// all groups are lifted by one batched call
int hb_rotate_sum_grouped(hb_ctx *c, const hb_ct *x, const int64_t *steps, int groups, hb_ct **out) {
    return guard(c, [&] {
        if (!x || !steps || groups < 1 || groups > 32) fail(HB_E_LIMIT, "rotate_sum: 1 to 32 terms");
        own(c, x);
        if (x->np != 2 || x->batch % groups) fail(HB_E_SHAPE, "rotate_sum: the batch does not split into that many groups");
        const int level = x->level, batch = x->batch / groups, N = c->N;
        const PlanDims d = plan_dims(c, level);
        const size_t ct_outer = (size_t)2 * d.n * N, dt_stride = (size_t)batch * d.dt_count * N;
        std::vector<const u64 *> base((size_t)groups);
        for (int t = 0; t < groups; ++t) base[(size_t)t] = x->d + (size_t)t * batch * ct_outer;
        Tmp dt(c, (size_t)x->batch * d.dt_count);
        ks_decompose(c, x->d + (size_t)d.n * N, ct_outer, level, x->batch, dt.p);
        *out = rotate_sum_core(c, base.data(), steps, groups, level, batch, x->spow, dt.p, dt_stride);
    });
}
int hb_rotate(hb_ctx *c, const hb_ct *a, int64_t steps, hb_ct **out) { return guard(c, [&] { *out = do_galois(c, a, c->h->galois_rot(steps)); }); }
int hb_conjugate(hb_ctx *c, const hb_ct *a, hb_ct **out) { return guard(c, [&] { *out = do_galois(c, a, c->h->galois_conj()); }); }
int hb_ntt(hb_ctx *c, hb_ct *a, int inverse) { return guard(c, [&] { own(c, a); ntt_inplace(c, a->d, (int)a->limbs(), c->qmap(a->level), inverse != 0); }); }

int hb_mul_pt_sum_parts(hb_ctx *c, const hb_ct *const *a, const hb_pt *const *p, int count, int parts, hb_ct **out) {
    return guard(c, [&] {
        if (!a || !p) fail(HB_E_ARG, "product sums: null argument");
        *out = do_prod_rescale_parts(c, a, p, count, parts);
    });
}
int hb_mul2_add_rescale(hb_ctx *c, const hb_ct *a, const hb_pt *pa, const hb_ct *b, const hb_pt *pb, hb_ct **out) {
    return guard(c, [&] {
        const hb_ct *as[2] = {a, b};
        const hb_pt *ps[2] = {pa, pb};
        *out = do_prod_rescale(c, as, ps, 2, false);
    });
}
int hb_matmul_acc_multi(hb_ctx *c, const hb_ct *pre, int btotal, int b0, const hb_pt *const *pts, int bcount, int64_t row_step, hb_ct **out) {
    return guard(c, [&] {
        if (btotal < 1 || pre->batch % btotal || b0 < 0 || bcount < 1 || b0 + bcount > btotal || bcount > 16) fail(HB_E_SHAPE, "matmul_acc: group selection");
        if (pre->np != 2 || pre->spow != 1) fail(HB_E_SHAPE, "matmul_acc: operands");
        own(c, pre);
        PtList pl{};
        for (int b = 0; b < bcount; ++b) {
            if (pre->level != pts[b]->level) fail(HB_E_LEVEL, "matmul_acc: plaintext level differs from the ciphertexts'");
            own(c, pts[b]);
            if (pts[b]->spow != 1) fail(HB_E_SHAPE, "matmul_acc: operands");
            pl.p[b] = pts[b]->d;
        }
        const int n = pre->level + 1, kc = pre->batch / btotal;
        const u32 *dg = galois_table(c, kc, row_step);
        hb_ct *r = new_ct(c, pre->level, 2, 1, 2);
        ALG(c, (size_t)kc * bcount * 2 * n + (size_t)bcount * n + 2 * n);
        LAUNCH(c), k_matmul_acc<<<c->egrid(2 * n), 256, 0, c->st>>>(r->d, pre->d, kc, btotal, b0, bcount, pl, dg, n, c->qmap(pre->level), c->pc, c->logn, c->N);
        *out = r;
    });
}
// `tiles` outputs from the same shifted copies: out[t] = sum over the groups b of matmul(copies of input b0 + b, pts[t * bcount + b])
int hb_matmul_acc_tiles(hb_ctx *c, const hb_ct *pre, int btotal, int b0, const hb_pt *const *pts, int bcount, int tiles, int64_t row_step, hb_ct **out) {
    return guard(c, [&] {
        if (!pre || !pts || !out || tiles < 1) fail(HB_E_ARG, "matmul_acc: null argument");
        if (btotal < 1 || pre->batch % btotal || b0 < 0 || bcount < 1 || b0 + bcount > btotal || bcount > 16) fail(HB_E_SHAPE, "matmul_acc: group selection");
        if (pre->np != 2 || pre->spow != 1) fail(HB_E_SHAPE, "matmul_acc: operands");
        own(c, pre);
        for (int i = 0; i < tiles * bcount; ++i) {
            if (!pts[i]) fail(HB_E_ARG, "matmul_acc: null plaintext");
            own(c, pts[i]);
            if (pre->level != pts[i]->level) fail(HB_E_LEVEL, "matmul_acc: plaintext level differs from the ciphertexts'");
            if (pts[i]->spow != 1) fail(HB_E_SHAPE, "matmul_acc: operands");
        }
        if (c->N % 512) { // small rings: tile by tile
            for (int t = 0; t < tiles; ++t) {
                int rc = hb_matmul_acc_multi(c, pre, btotal, b0, pts + (size_t)t * bcount, bcount, row_step, &out[t]);
                if (rc != HB_OK) { for (int u = 0; u < t; ++u) { hb_ct_free(out[u]); out[u] = nullptr; } throw ArgFail{rc, c->err}; }
            }
            return;
        }
        const int n = pre->level + 1, kc = pre->batch / btotal;
        const u32 *dg = galois_table(c, kc, row_step);
        std::vector<hb_ct *> rs((size_t)tiles, nullptr);
        try {
            for (int t = 0; t < tiles; ++t) rs[(size_t)t] = new_ct(c, pre->level, 2, 1, 2);
            ALG(c, (size_t)kc * bcount * 2 * n + (size_t)tiles * ((size_t)bcount * n + 2 * n));
            int t = 0;
            while (t < tiles) {
                const int left = tiles - t;
                if (left >= 4) { launch_matmul_tiles<4>(c, pre, btotal, b0, pts + (size_t)t * bcount, bcount, kc, dg, rs.data() + t); t += 4; }
                else if (left == 3) { launch_matmul_tiles<3>(c, pre, btotal, b0, pts + (size_t)t * bcount, bcount, kc, dg, rs.data() + t); t += 3; }
                else if (left == 2) { launch_matmul_tiles<2>(c, pre, btotal, b0, pts + (size_t)t * bcount, bcount, kc, dg, rs.data() + t); t += 2; }
                else { launch_matmul_tiles<1>(c, pre, btotal, b0, pts + (size_t)t * bcount, bcount, kc, dg, rs.data() + t); t += 1; }
            }
            CK(cudaGetLastError());
        } catch (...) { for (hb_ct *r : rs) if (r) hb_ct_free(r); throw; }
        for (int t = 0; t < tiles; ++t) out[t] = rs[(size_t)t];
    });
}
int hb_matmul_acc(hb_ctx *c, const hb_ct *pre, const hb_pt *pt, int64_t row_step, hb_ct **out) { return hb_matmul_acc_multi(c, pre, 1, 0, &pt, 1, row_step, out); }
int hb_pt_rotate(hb_ctx *c, const hb_pt *p, int64_t steps, hb_pt **out) {
    return guard(c, [&] {
        hb_pt *r = new_pt(c, p->level, p->spow);
        const u64 g = c->h->galois_rot(steps);
        if (g == 1) CK(cudaMemcpyAsync(r->d, p->d, (size_t)(p->level + 1) * c->N * 8, cudaMemcpyDeviceToDevice, c->st));
        else LAUNCH(c), k_permute<<<c->egrid(p->level + 1), 256, 0, c->st>>>(r->d, p->d, (u32)g, c->logn, c->N);
        *out = r;
    });
}
// plaintext x plaintext with rescale, and plaintext + plaintext: a plaintext is handled as a one-polynomial ciphertext
int hb_pt_mul(hb_ctx *c, const hb_pt *a, const hb_pt *b, hb_pt **out) {
    return guard(c, [&] {
        hb_ct view{c, a->level, 1, 1, a->spow, a->d};
        const hb_ct *vp = &view;
        hb_ct *r = do_prod_rescale(c, &vp, &b, 1, true);
        hb_pt *p = new hb_pt{c, r->level, 1, r->d};
        delete r; // the buffer now belongs to the plaintext handle
        *out = p;
    });
}
int hb_pt_add(hb_ctx *c, const hb_pt *a, const hb_pt *b, hb_pt **out) {
    return guard(c, [&] {
        if (a->level != b->level) fail(HB_E_LEVEL, "pt_add: level mismatch");
        if (a->spow != b->spow) fail(HB_E_SHAPE, "pt_add: scale mismatch");
        hb_pt *r = new_pt(c, a->level, a->spow);
        LAUNCH(c), k_addsub<<<c->egrid(a->level + 1), 256, 0, c->st>>>(r->d, a->d, b->d, c->qmap(a->level), c->pc, c->N, 0);
        *out = r;
    });
}
int hb_mod_reduce(hb_ctx *c, hb_ct *a) {
    return guard(c, [&] {
        own(c, a);
        LAUNCH(c), k_mod_reduce<<<c->egrid((int)a->limbs()), 256, 0, c->st>>>(a->d, c->qmap(a->level), c->pc, c->N);
    });
}
// out = (sum of the parts) mod q, one pass: the owner's half of a K-split exchange (its own partial product plus the
// ones received from the other ranks).  Parts hold canonical residues; at most 16 of them.
int hb_sum_mod_reduce(hb_ctx *c, const hb_ct *const *parts, int count, hb_ct **out) {
    return guard(c, [&] {
        if (!parts || count < 1 || count > 16) fail(HB_E_LIMIT, "sum_mod_reduce: 1 to 16 parts");
        SumList sl{}; sl.count = count;
        for (int t = 0; t < count; ++t) {
            own(c, parts[t]);
            check_same(parts[0], parts[t], "sum_mod_reduce");
            sl.x[t] = parts[t]->d;
        }
        hb_ct *r = new_ct(c, parts[0]->level, parts[0]->np, parts[0]->batch, parts[0]->spow);
        ALG(c, (size_t)(count + 1) * r->limbs());
        LAUNCH(c), k_sum_mod<<<c->egrid((int)r->limbs()), 256, 0, c->st>>>(r->d, sl, c->qmap(r->level), c->pc, c->N);
        *out = r;
    });
}
// Sum over ranks of residues below 2^60 cannot overflow 64 bits for up to 16 ranks; the owner
// reduces afterwards (same order of operations as HEMMer::ncclAllReduceWrapper + modReduct).
int hb_allreduce_sum(hb_ctx *c, hb_ct *a, void *comm) {
    return guard(c, [&] {
        own(c, a);
        const NcclApi &nc = nccl_api();
        if (!nc.ok) fail(HB_E_NCCL, "NCCL library not available");
        ncclResult_t r = nc.AllReduce(a->d, a->d, a->limbs() * c->N, ncclUint64, ncclSum, (ncclComm_t)comm, c->st);
        if (r != ncclSuccess) fail(HB_E_NCCL, nc.GetErrorString(r));
        LAUNCH(c), k_mod_reduce<<<c->egrid((int)a->limbs()), 256, 0, c->st>>>(a->d, c->qmap(a->level), c->pc, c->N);
    });
}
// Sum to one owner: TransformerBlock::ncclReduceWrapper / ncclReduceWrapperHidden (ncclReduce to `root`), followed on
// the root by the reduction modulo each prime.  The other ranks' buffers are left as they were.
int hb_reduce_sum(hb_ctx *c, hb_ct *a, int root, int my_rank, void *comm) {
    return guard(c, [&] {
        own(c, a);
        const NcclApi &nc = nccl_api();
        if (!nc.ok) fail(HB_E_NCCL, "NCCL library not available");
        ncclResult_t r = nc.Reduce(a->d, a->d, a->limbs() * c->N, ncclUint64, ncclSum, root, (ncclComm_t)comm, c->st);
        if (r != ncclSuccess) fail(HB_E_NCCL, nc.GetErrorString(r));
        if (my_rank == root) LAUNCH(c), k_mod_reduce<<<c->egrid((int)a->limbs()), 256, 0, c->st>>>(a->d, c->qmap(a->level), c->pc, c->N);
    });
}
int hb_allgather(hb_ctx *c, const hb_ct *mine, hb_ct *all, void *comm) {
    return guard(c, [&] {
        own(c, mine, all);
        if (all->level != mine->level || all->np != mine->np || all->batch % mine->batch) fail(HB_E_SHAPE, "allgather: geometry");
        const NcclApi &nc = nccl_api();
        if (!nc.ok) fail(HB_E_NCCL, "NCCL library not available");
        ncclResult_t r = nc.AllGather(mine->d, all->d, mine->limbs() * c->N, ncclUint64, (ncclComm_t)comm, c->st);
        if (r != ncclSuccess) fail(HB_E_NCCL, nc.GetErrorString(r));
    });
}
// Point-to-point moves of whole handles, to be issued between hb_nccl_group_start and hb_nccl_group_end on both sides
// (every send needs its receive in the same group, as NCCL requires).
int hb_nccl_group_start() { const NcclApi &nc = nccl_api(); return nc.ok && nc.GroupStart() == ncclSuccess ? HB_OK : HB_E_NCCL; }
int hb_nccl_group_end() { const NcclApi &nc = nccl_api(); return nc.ok && nc.GroupEnd() == ncclSuccess ? HB_OK : HB_E_NCCL; }
int hb_send(hb_ctx *c, const hb_ct *a, int peer, void *comm) {
    return guard(c, [&] {
        own(c, a);
        const NcclApi &nc = nccl_api();
        if (!nc.ok) fail(HB_E_NCCL, "NCCL library not available");
        ncclResult_t r = nc.Send(a->d, a->limbs() * c->N, ncclUint64, peer, (ncclComm_t)comm, c->st);
        if (r != ncclSuccess) fail(HB_E_NCCL, nc.GetErrorString(r));
    });
}
int hb_recv(hb_ctx *c, hb_ct *a, int peer, void *comm) {
    return guard(c, [&] {
        own(c, a);
        const NcclApi &nc = nccl_api();
        if (!nc.ok) fail(HB_E_NCCL, "NCCL library not available");
        ncclResult_t r = nc.Recv(a->d, a->limbs() * c->N, ncclUint64, peer, (ncclComm_t)comm, c->st);
        if (r != ncclSuccess) fail(HB_E_NCCL, nc.GetErrorString(r));
    });
}
int hb_nccl_unique_id(void *id128) {
    const NcclApi &nc = nccl_api();
    if (!nc.ok || !id128) return HB_E_NCCL;
    ncclUniqueId id;
    if (nc.GetUniqueId(&id) != ncclSuccess) return HB_E_NCCL;
    std::memcpy(id128, &id, sizeof(id));
    return HB_OK;
}
int hb_nccl_comm_init(hb_ctx *c, int nranks, int rank, const void *id128, void **comm) {
    return guard(c, [&] {
        const NcclApi &nc = nccl_api();
        if (!nc.ok) fail(HB_E_NCCL, "NCCL library not available");
        ncclUniqueId id; std::memcpy(&id, id128, sizeof(id));
        ncclComm_t cm = nullptr;
        ncclResult_t r = nc.CommInitRank(&cm, nranks, id, rank);
        if (r != ncclSuccess) fail(HB_E_NCCL, nc.GetErrorString(r));
        *comm = cm;
    });
}
int hb_nccl_comm_destroy(void *comm) {
    const NcclApi &nc = nccl_api();
    if (!nc.ok) return HB_E_NCCL;
    return nc.CommDestroy((ncclComm_t)comm) == ncclSuccess ? HB_OK : HB_E_NCCL;
}


// ---- files ---------------------------------------------------------------------------------------------------
// One self-describing container for ciphertexts, plaintexts and keys (HEaaN's own binary format is not published, so
// files of the reference cannot be read; these take their place for the same calls: Ciphertext::save / load,
// HEMMer::save).  Layout, little-endian:
//     FileHeader (96 bytes) | payload: plain residues, uint64, in the device layout of the object | FNV-1a-64 of the payload
// A file is only accepted by a context with the same ring degree and the same primes (prime_hash).
namespace {
enum FileKind : uint32_t { kFileCt = 1, kFilePt = 2, kFileEvk = 3, kFileSecret = 4 };
struct FileHeader {
    char magic[8];          // "HB200F1\0"
    uint32_t kind, log_n, level, n_poly, batch, scale_pow, ext, digits, nprimes, reserved;
    uint64_t galois;        // switching keys: Galois element (0: multiplication key)
    uint64_t prime_hash;    // FNV-1a over the context's primes
    uint64_t payload_words;
    uint64_t reserved2[3];
};
static_assert(sizeof(FileHeader) == 96, "file header layout");
uint64_t fnv1a(const void *data, size_t bytes, uint64_t h = 1469598103934665603ull) {
    const unsigned char *p = (const unsigned char *)data;
    for (size_t i = 0; i < bytes; ++i) { h ^= p[i]; h *= 1099511628211ull; }
    return h;
}
uint64_t prime_hash(const hb_ctx *c) { return fnv1a(c->h->q.data(), c->h->q.size() * 8); }
struct File {
    FILE *f;
    File(const char *path, const char *mode) : f(path ? std::fopen(path, mode) : nullptr) { if (!f) fail(HB_E_ARG, std::string("cannot open ") + (path ? path : "(null)")); }
    ~File() { if (f) std::fclose(f); }
};
void write_file(hb_ctx *c, const char *path, FileHeader h, const u64 *dev, size_t words) {
    no_capture(c, "save");
    std::vector<u64> host(words);
    CK(cudaMemcpyAsync(host.data(), dev, words * 8, cudaMemcpyDeviceToHost, c->st));
    CK(cudaStreamSynchronize(c->st));
    std::memcpy(h.magic, "HB200F1", 8);
    h.log_n = (uint32_t)c->logn; h.nprimes = (uint32_t)c->nprimes; h.prime_hash = prime_hash(c); h.payload_words = words;
    const uint64_t sum = fnv1a(host.data(), words * 8);
    File out(path, "wb");
    if (std::fwrite(&h, sizeof(h), 1, out.f) != 1 || std::fwrite(host.data(), 8, words, out.f) != words || std::fwrite(&sum, 8, 1, out.f) != 1)
        fail(HB_E_ARG, std::string("short write to ") + path);
}
// reads header + payload; checks magic, kind, context and checksum
std::vector<u64> read_file(hb_ctx *c, const char *path, uint32_t kind, FileHeader &h) {
    File in(path, "rb");
    if (std::fread(&h, sizeof(h), 1, in.f) != 1 || std::memcmp(h.magic, "HB200F1", 8) != 0) fail(HB_E_ARG, std::string(path) + ": not a file of this library");
    if (h.kind != kind) fail(HB_E_ARG, std::string(path) + ": holds another kind of object");
    if (h.log_n != (uint32_t)c->logn || h.nprimes != (uint32_t)c->nprimes || h.prime_hash != prime_hash(c)) fail(HB_E_ARG, std::string(path) + ": written under other parameters");
    if (h.payload_words > ((uint64_t)1 << 34)) fail(HB_E_LIMIT, std::string(path) + ": implausible size");
    std::vector<u64> host((size_t)h.payload_words);
    uint64_t sum = 0;
    if (std::fread(host.data(), 8, host.size(), in.f) != host.size() || std::fread(&sum, 8, 1, in.f) != 1) fail(HB_E_ARG, std::string(path) + ": truncated");
    if (sum != fnv1a(host.data(), host.size() * 8)) fail(HB_E_ARG, std::string(path) + ": checksum mismatch");
    return host;
}
void upload(hb_ctx *c, u64 *dev, const std::vector<u64> &host) {
    CK(cudaMemcpyAsync(dev, host.data(), host.size() * 8, cudaMemcpyHostToDevice, c->st));
    CK(cudaStreamSynchronize(c->st));
}
void save_evk(hb_ctx *c, const Evk &k, uint64_t g, const std::string &path) {
    const size_t limbs = (size_t)k.nd * 2 * c->nprimes;
    FileHeader h{}; h.kind = kFileEvk; h.level = (uint32_t)c->L; h.digits = (uint32_t)k.nd; h.galois = g; h.n_poly = 2;
    write_file(c, path.c_str(), h, k.d, limbs * c->N);
}
} // namespace

// Ciphertext::save / load (Ciphertext.hpp:89-98), used by the reference to carry activations from the forward to the
// backward pass (HEMMer.cpp:1403-1405, TransformerBlock.cpp:11059-11079)
int hb_ct_save(hb_ctx *c, const hb_ct *x, const char *path) {
    return guard(c, [&] {
        own(c, x);
        FileHeader h{}; h.kind = kFileCt; h.level = (uint32_t)x->level; h.n_poly = (uint32_t)x->np; h.batch = (uint32_t)x->batch; h.scale_pow = (uint32_t)x->spow;
        write_file(c, path, h, x->d, x->limbs() * c->N);
    });
}
int hb_ct_load(hb_ctx *c, const char *path, hb_ct **out) {
    return guard(c, [&] {
        no_capture(c, "load");
        FileHeader h;
        const std::vector<u64> host = read_file(c, path, kFileCt, h);
        hb_ct *r = new_ct(c, (int)h.level, (int)h.n_poly, (int)h.batch, (int)h.scale_pow);
        if (r->limbs() * c->N != host.size()) { hb_ct_free(r); fail(HB_E_ARG, std::string(path) + ": size does not match its header"); }
        try { upload(c, r->d, host); } catch (...) { hb_ct_free(r); throw; }
        *out = r;
    });
}
// Plaintext::save / load (Plaintext.hpp), e.g. the encoded weights the reference writes once and reloads (HEMMer::encodeWeight)
int hb_pt_save(hb_ctx *c, const hb_pt *x, const char *path) {
    return guard(c, [&] {
        own(c, x);
        FileHeader h{}; h.kind = kFilePt; h.level = (uint32_t)x->level; h.scale_pow = (uint32_t)x->spow; h.ext = (uint32_t)x->ext; h.n_poly = 1; h.batch = 1;
        write_file(c, path, h, x->d, (size_t)(x->level + 1 + (x->ext ? c->K : 0)) * c->N);
    });
}
int hb_pt_load(hb_ctx *c, const char *path, hb_pt **out) {
    return guard(c, [&] {
        no_capture(c, "load");
        FileHeader h;
        const std::vector<u64> host = read_file(c, path, kFilePt, h);
        const size_t limbs = (size_t)h.level + 1 + (h.ext ? c->K : 0);
        if ((int)h.level > c->L || limbs * c->N != host.size()) fail(HB_E_ARG, std::string(path) + ": size does not match its header");
        hb_pt *r = new hb_pt{c, (int)h.level, (int)h.scale_pow, nullptr};
        r->ext = h.ext ? 1 : 0;
        try { r->d = c->alloc_limbs(limbs); upload(c, r->d, host); } catch (...) { if (r->d) c->pool.put(r->d); delete r; throw; }
        *out = r;
    });
}
// HEMMer::save (HEMMer.cpp:225-230): SecretKey.bin plus the key pack -- here MultKey.bin and one GaloisKey_<g>.bin per
// generated rotation / conjugation key -- under an existing directory
int hb_keys_save(hb_ctx *c, const char *dir) {
    return guard(c, [&] {
        if (!dir) fail(HB_E_ARG, "keys_save: null path");
        if (!c->have_sk) fail(HB_E_NOKEY, "secret key not generated");
        const std::string d(dir);
        FileHeader h{}; h.kind = kFileSecret; h.level = (uint32_t)c->L; h.n_poly = 1;
        write_file(c, (d + "/SecretKey.bin").c_str(), h, c->sk, (size_t)c->nprimes * c->N);
        if (c->mult_key.d) save_evk(c, c->mult_key, 0, d + "/MultKey.bin");
        for (const auto &kv : c->gal_keys) save_evk(c, kv.second, kv.first, d + "/GaloisKey_" + std::to_string(kv.first) + ".bin");
    });
}
// the reverse: secret key, multiplication key and the Galois keys named by `galois` (count entries) from `dir`
int hb_keys_load(hb_ctx *c, const char *dir, const uint64_t *galois, int count) {
    return guard(c, [&] {
        no_capture(c, "load");
        if (!dir || count < 0 || (count && !galois)) fail(HB_E_ARG, "keys_load: bad arguments");
        const std::string d(dir);
        FileHeader h;
        std::vector<u64> host = read_file(c, (d + "/SecretKey.bin").c_str(), kFileSecret, h);
        if (host.size() != (size_t)c->nprimes * c->N) fail(HB_E_ARG, "SecretKey.bin: size does not match the context");
        upload(c, c->sk, host);
        c->have_sk = true;
        auto load_evk = [&](const std::string &path, uint64_t g) {
            std::vector<u64> w = read_file(c, path.c_str(), kFileEvk, h);
            const int nd = c->h->digit_of(c->h->L) + 1;
            const size_t limbs = (size_t)nd * 2 * c->nprimes;
            if ((int)h.digits != nd || h.galois != g || w.size() != limbs * c->N) fail(HB_E_ARG, path + ": does not fit this context");
            Evk k; k.nd = nd; k.d = c->alloc_limbs(limbs);
            try { upload(c, k.d, w); } catch (...) { c->pool.put(k.d); throw; }
            return k;
        };
        auto replace = [&](Evk &slot, Evk k) { if (slot.d) c->pool.put(slot.d); slot = k; };
        replace(c->mult_key, load_evk(d + "/MultKey.bin", 0));
        for (int i = 0; i < count; ++i) replace(c->gal_keys[galois[i]], load_evk(d + "/GaloisKey_" + std::to_string(galois[i]) + ".bin", galois[i]));
    });
}

int hb_set_host_threads(hb_ctx *c, int n) { if (!c || n < 0) return HB_E_ARG; c->host_threads = n; return HB_OK; }

// ---- CUDA graph of a fixed launch sequence -------------------------------------------------------------------
// Between hb_graph_begin and hb_graph_end the calls made on this context are recorded instead of run.  The pool hands
// out the same buffers as in any other pass, so the recorded kernels read and write fixed addresses: the caller keeps
// the operand handles alive and unchanged in place, and keeps the result handles of the recorded pass for as long as
// it replays the graph (every replay writes the results into those same buffers).  Everything the pass needs that is
// made on first use -- rotation keys, plans, masks, masked keys, Galois tables, pool buffers -- must exist already:
// run the pass once before recording it.  Calls that copy to or from the host are refused while recording.
struct hb_graph { hb_ctx *ctx; cudaGraph_t g; cudaGraphExec_t e; unsigned long long kernels, alg_limbs; };
int hb_graph_begin(hb_ctx *c) {
    return guard(c, [&] {
        if (c->capturing) fail(HB_E_ARG, "graph: already recording");
        CK(cudaStreamBeginCapture(c->st, cudaStreamCaptureModeRelaxed));
        c->capturing = true;
        c->launches_at_capture = c->launches;
        c->alg_at_capture = c->alg_limbs;
    });
}
int hb_graph_end(hb_ctx *c, hb_graph **out) {
    return guard(c, [&] {
        if (!c->capturing) fail(HB_E_ARG, "graph: not recording");
        c->capturing = false;
        cudaGraph_t g = nullptr;
        CK(cudaStreamEndCapture(c->st, &g));
        cudaGraphExec_t e = nullptr;
        cudaError_t rc = cudaGraphInstantiate(&e, g, 0);
        if (rc != cudaSuccess) { cudaGraphDestroy(g); throw CudaFail{rc, "cudaGraphInstantiate"}; }
        *out = new hb_graph{c, g, e, c->launches - c->launches_at_capture, c->alg_limbs - c->alg_at_capture};
    });
}
int hb_graph_launch(hb_ctx *c, hb_graph *g) {
    return guard(c, [&] {
        if (!g || g->ctx != c) fail(HB_E_ARG, "graph belongs to another context");
        CK(cudaGraphLaunch(g->e, c->st));
        c->launches += g->kernels;
        c->alg_limbs += g->alg_limbs;
    });
}
uint64_t hb_graph_kernels(const hb_graph *g) { return g ? g->kernels : 0; }
void hb_graph_free(hb_graph *g) {
    if (!g) return;
    cudaSetDevice(g->ctx->device);
    cudaGraphExecDestroy(g->e); cudaGraphDestroy(g->g);
    delete g;
}

} // extern "C"
