// Negacyclic NTT / inverse NTT over RNS limbs for sm_100a.
//
// Output order of the forward transform: a_hat[i] = a(psi^(2*bitrev(i)+1)); twiddle tables hold
// psi^bitrev(k) (forward) and psi^-bitrev(k) (inverse) with their Shoup companions.
//
// N = 2^16 path: the limb is a 256 x 256 matrix (index = row*256 + col).  The forward transform
// is a column pass (stages 1-8, butterfly distance >= 256) followed by a row pass (stages 9-16);
// the inverse runs the row pass first.  Each pass moves a limb through HBM once: a CTA of 256
// threads owns 16 columns (or 16 rows), every thread keeps 16 coefficients in registers and
// performs four butterfly stages at a time (radix 16), exchanging through shared memory once.
// Global accesses are 128-byte runs per half-warp in both passes.
//
// N <= 4096 path (used by small-parameter tests): one CTA transforms a whole limb in shared memory.
#pragma once
#include "modarith.cuh"

namespace hb {

struct NttTables {
    const u64 *psi, *psi_sh, *ipsi, *ipsi_sh; // each [nprimes][N]
};

// address of limb instance li: (li / map.n) * outer + (li % map.n) * N
struct LimbAddr {
    size_t outer;
    __device__ __forceinline__ size_t off(int li, int period, int N) const {
        return (size_t)(li / period) * outer + (size_t)(li % period) * N;
    }
};

__device__ __forceinline__ void ct_bfly(u64 &x, u64 &y, u64 w, u64 ws, u64 q, u64 q2) {
    x = x >= q2 ? x - q2 : x;
    u64 t = mul_shoup_lazy(y, w, ws, q);
    y = x + q2 - t;
    x = x + t;
}
__device__ __forceinline__ void gs_bfly(u64 &x, u64 &y, u64 w, u64 ws, u64 q, u64 q2) {
    u64 s = x + y;
    u64 d = x + q2 - y;
    x = s >= q2 ? s - q2 : s;
    y = mul_shoup_lazy(d, w, ws, q);
}

// four Cooley-Tukey stages on 16 register values; local stage s, group g uses twiddle (base<<s)+g
__device__ __forceinline__ void fwd16(u64 (&v)[16], const u64 *__restrict__ w, const u64 *__restrict__ ws, u32 base, u64 q) {
    const u64 q2 = q << 1;
#pragma unroll
    for (int s = 0; s < 4; ++s) {
        const int half = 8 >> s;
#pragma unroll
        for (int g = 0; g < (1 << s); ++g) {
            const u64 tw = __ldg(w + ((base << s) + g)), tws = __ldg(ws + ((base << s) + g));
#pragma unroll
            for (int j = 0; j < half; ++j) ct_bfly(v[g * 2 * half + j], v[g * 2 * half + j + half], tw, tws, q, q2);
        }
    }
}
// four Gentleman-Sande stages, the mirror image of fwd16
__device__ __forceinline__ void inv16(u64 (&v)[16], const u64 *__restrict__ w, const u64 *__restrict__ ws, u32 base, u64 q) {
    const u64 q2 = q << 1;
#pragma unroll
    for (int s = 3; s >= 0; --s) {
        const int half = 8 >> s;
#pragma unroll
        for (int g = 0; g < (1 << s); ++g) {
            const u64 tw = __ldg(w + ((base << s) + g)), tws = __ldg(ws + ((base << s) + g));
#pragma unroll
            for (int j = 0; j < half; ++j) gs_bfly(v[g * 2 * half + j], v[g * 2 * half + j + half], tw, tws, q, q2);
        }
    }
}

// ---- small-prime variants: the second twiddle table holds w/q as a double ----
// forward: values only grow by < 1.6q per stage (canonical input, 16 stages: < 27q < 2^47), no corrections
__device__ __forceinline__ void ct_bfly_fp(u64 &x, u64 &y, u64 w, double wf, u64 q, u64 q2) {
    const u64 t = mul_fp_lazy(y, w, wf, q);
    y = x + q2 - t;
    x = x + t;
}
// inverse: the sum path doubles per stage, so callers reduce every four stages; `off` is a multiple of q
// above the largest y of the stage
__device__ __forceinline__ void gs_bfly_fp(u64 &x, u64 &y, u64 w, double wf, u64 q, u64 off) {
    const u64 s = x + y;
    const u64 d = x + off - y;
    x = s;
    y = mul_fp_lazy(d, w, wf, q);
}
__device__ __forceinline__ void fwd16_fp(u64 (&v)[16], const u64 *__restrict__ w, const double *__restrict__ wf, u32 base, u64 q) {
    const u64 q2 = q << 1;
#pragma unroll
    for (int s = 0; s < 4; ++s) {
        const int half = 8 >> s;
#pragma unroll
        for (int g = 0; g < (1 << s); ++g) {
            const u64 tw = __ldg(w + ((base << s) + g));
            const double twf = __ldg(wf + ((base << s) + g));
#pragma unroll
            for (int j = 0; j < half; ++j) ct_bfly_fp(v[g * 2 * half + j], v[g * 2 * half + j + half], tw, twf, q, q2);
        }
    }
}
// inputs below 2q; outputs below 32q (sum path) -- reduce before the next round
__device__ __forceinline__ void inv16_fp(u64 (&v)[16], const u64 *__restrict__ w, const double *__restrict__ wf, u32 base, u64 q) {
#pragma unroll
    for (int s = 3; s >= 0; --s) {
        const int half = 8 >> s;
        const u64 off = q << (4 - s); // inputs of local stage s are below 2q * 2^(3-s)
#pragma unroll
        for (int g = 0; g < (1 << s); ++g) {
            const u64 tw = __ldg(w + ((base << s) + g));
            const double twf = __ldg(wf + ((base << s) + g));
#pragma unroll
            for (int j = 0; j < half; ++j) gs_bfly_fp(v[g * 2 * half + j], v[g * 2 * half + j + half], tw, twf, q, off);
        }
    }
}

constexpr int kN16 = 65536;
constexpr int kRowStride = 272; // 256 + one pad word per 16: conflict-free 16-consecutive reads

// ---- forward, column pass: stages 1..8.  Output range [0, 4q). ----
__global__ void __launch_bounds__(256, 4) ntt16_fwd_cols(const u64 *__restrict__ src, LimbAddr sa, u64 *__restrict__ dst, LimbAddr da,
                                                      LimbMap map, const PrimeConst *__restrict__ pc, NttTables tb) {
    __shared__ u64 sm[4096];
    const int li = blockIdx.y, pi = map.prime[li % map.n];
    const u64 q = pc[pi].q;
    const u64 *w = tb.psi + (size_t)pi * kN16, *ws = tb.psi_sh + (size_t)pi * kN16;
    const int tid = threadIdx.x, lane = tid & 15, sub = tid >> 4;
    const u64 *p = src + sa.off(li, map.n, kN16) + blockIdx.x * 16 + lane;
    u64 *o = dst + da.off(li, map.n, kN16) + blockIdx.x * 16 + lane;
    const bool fp = pc[pi].small != 0;
    const double *wf = reinterpret_cast<const double *>(ws);
    u64 v[16];
#pragma unroll
    for (int e = 0; e < 16; ++e) v[e] = p[(e * 16 + sub) * 256];
    if (fp) fwd16_fp(v, w, wf, 1u, q); else fwd16(v, w, ws, 1u, q);
#pragma unroll
    for (int e = 0; e < 16; ++e) sm[(e * 16 + sub) * 16 + lane] = v[e];
    __syncthreads();
#pragma unroll
    for (int e = 0; e < 16; ++e) v[e] = sm[(sub * 16 + e) * 16 + lane];
    if (fp) fwd16_fp(v, w, wf, 16u + sub, q); else fwd16(v, w, ws, 16u + sub, q);
#pragma unroll
    for (int e = 0; e < 16; ++e) o[(sub * 16 + e) * 256] = v[e];
}

// ---- forward, row pass: stages 9..16.  Input [0, 4q), output canonical [0, q). ----
__global__ void __launch_bounds__(256, 4) ntt16_fwd_rows(const u64 *__restrict__ src, LimbAddr sa, u64 *__restrict__ dst, LimbAddr da,
                                                      LimbMap map, const PrimeConst *__restrict__ pc, NttTables tb) {
    __shared__ u64 sm[16 * kRowStride];
    const int li = blockIdx.y, pi = map.prime[li % map.n];
    const u64 q = pc[pi].q, q2 = q << 1;
    const u64 *w = tb.psi + (size_t)pi * kN16, *ws = tb.psi_sh + (size_t)pi * kN16;
    const int tid = threadIdx.x, clo = tid & 15, rl = tid >> 4;
    const int row = blockIdx.x * 16 + rl;
    const u64 *p = src + sa.off(li, map.n, kN16) + (size_t)row * 256 + clo;
    u64 *o = dst + da.off(li, map.n, kN16) + (size_t)row * 256 + clo;
    u64 *smr = sm + rl * kRowStride;
    const bool fp = pc[pi].small != 0;
    const double *wf = reinterpret_cast<const double *>(ws);
    const double qinv = pc[pi].q_inv_f;
    u64 v[16];
#pragma unroll
    for (int e = 0; e < 16; ++e) v[e] = p[e * 16];
    if (fp) fwd16_fp(v, w, wf, 256u + row, q); else fwd16(v, w, ws, 256u + row, q);
#pragma unroll
    for (int e = 0; e < 16; ++e) smr[e * 17 + clo] = v[e];
    __syncthreads();
#pragma unroll
    for (int e = 0; e < 16; ++e) v[e] = smr[clo * 17 + e];
    if (fp) fwd16_fp(v, w, wf, ((256u + row) << 4) + clo, q); else fwd16(v, w, ws, ((256u + row) << 4) + clo, q);
#pragma unroll
    for (int e = 0; e < 16; ++e) {
        u64 x = v[e];
        if (fp) x = reduce_fp(x, qinv, q);
        else { x = x >= q2 ? x - q2 : x; x = x >= q ? x - q : x; }
        smr[clo * 17 + e] = x;
    }
    __syncthreads();
#pragma unroll
    for (int e = 0; e < 16; ++e) o[e * 16] = smr[e * 17 + clo];
}

// ---- inverse, row pass: undoes stages 16..9.  Input canonical, output [0, 2q). ----
__global__ void __launch_bounds__(256, 4) ntt16_inv_rows(const u64 *__restrict__ src, LimbAddr sa, u64 *__restrict__ dst, LimbAddr da,
                                                      LimbMap map, const PrimeConst *__restrict__ pc, NttTables tb) {
    __shared__ u64 sm[16 * kRowStride];
    const int li = blockIdx.y, pi = map.prime[li % map.n];
    const u64 q = pc[pi].q;
    const u64 *w = tb.ipsi + (size_t)pi * kN16, *ws = tb.ipsi_sh + (size_t)pi * kN16;
    const int tid = threadIdx.x, clo = tid & 15, rl = tid >> 4;
    const int row = blockIdx.x * 16 + rl;
    const u64 *p = src + sa.off(li, map.n, kN16) + (size_t)row * 256 + clo;
    u64 *o = dst + da.off(li, map.n, kN16) + (size_t)row * 256 + clo;
    u64 *smr = sm + rl * kRowStride;
    u64 v[16];
#pragma unroll
    for (int e = 0; e < 16; ++e) smr[e * 17 + clo] = p[e * 16];
    __syncthreads();
    const bool fp = pc[pi].small != 0;
    const double *wf = reinterpret_cast<const double *>(ws);
    const double qinv = pc[pi].q_inv_f;
#pragma unroll
    for (int e = 0; e < 16; ++e) v[e] = smr[clo * 17 + e];
    if (fp) {
        inv16_fp(v, w, wf, ((256u + row) << 4) + clo, q);
#pragma unroll
        for (int e = 0; e < 16; ++e) v[e] = reduce_fp_lazy(v[e], qinv, q);
    } else inv16(v, w, ws, ((256u + row) << 4) + clo, q);
#pragma unroll
    for (int e = 0; e < 16; ++e) smr[clo * 17 + e] = v[e];
    __syncthreads();
#pragma unroll
    for (int e = 0; e < 16; ++e) v[e] = smr[e * 17 + clo];
    if (fp) {
        inv16_fp(v, w, wf, 256u + row, q);
#pragma unroll
        for (int e = 0; e < 16; ++e) v[e] = reduce_fp_lazy(v[e], qinv, q);
    } else inv16(v, w, ws, 256u + row, q);
#pragma unroll
    for (int e = 0; e < 16; ++e) o[e * 16] = v[e];
}

// ---- inverse, column pass: undoes stages 8..1, scales by N^-1.  Input [0, 2q), output canonical. ----
__global__ void __launch_bounds__(256, 4) ntt16_inv_cols(const u64 *__restrict__ src, LimbAddr sa, u64 *__restrict__ dst, LimbAddr da,
                                                      LimbMap map, const PrimeConst *__restrict__ pc, NttTables tb) {
    __shared__ u64 sm[4096];
    const int li = blockIdx.y, pi = map.prime[li % map.n];
    const u64 q = pc[pi].q;
    const u64 ninv = pc[pi].n_inv, ninv_sh = pc[pi].n_inv_sh;
    const u64 *w = tb.ipsi + (size_t)pi * kN16, *ws = tb.ipsi_sh + (size_t)pi * kN16;
    const int tid = threadIdx.x, lane = tid & 15, sub = tid >> 4;
    const u64 *p = src + sa.off(li, map.n, kN16) + blockIdx.x * 16 + lane;
    u64 *o = dst + da.off(li, map.n, kN16) + blockIdx.x * 16 + lane;
    const bool fp = pc[pi].small != 0;
    const double *wf = reinterpret_cast<const double *>(ws);
    const double qinv = pc[pi].q_inv_f, ninv_f = pc[pi].n_inv_f;
    u64 v[16];
#pragma unroll
    for (int e = 0; e < 16; ++e) v[e] = p[(sub * 16 + e) * 256];
    if (fp) {
        inv16_fp(v, w, wf, 16u + sub, q);
#pragma unroll
        for (int e = 0; e < 16; ++e) v[e] = reduce_fp_lazy(v[e], qinv, q);
    } else inv16(v, w, ws, 16u + sub, q);
#pragma unroll
    for (int e = 0; e < 16; ++e) sm[(sub * 16 + e) * 16 + lane] = v[e];
    __syncthreads();
#pragma unroll
    for (int e = 0; e < 16; ++e) v[e] = sm[(e * 16 + sub) * 16 + lane];
    if (fp) {
        inv16_fp(v, w, wf, 1u, q);
#pragma unroll
        for (int e = 0; e < 16; ++e) {
            // x * N^-1: quotient from the FP64 pipe, remainder in (-0.6q, 0.6q) shifted by q, then canonical
            u64 r = mul_fp_lazy(v[e], ninv, ninv_f, q);
            o[(e * 16 + sub) * 256] = r >= q ? r - q : r;
        }
    } else {
        inv16(v, w, ws, 1u, q);
#pragma unroll
        for (int e = 0; e < 16; ++e) o[(e * 16 + sub) * 256] = mul_shoup(v[e], ninv, ninv_sh, q);
    }
}

// ---- whole limb in shared memory, N <= 4096 ----
__global__ void __launch_bounds__(256) ntt_small(const u64 *__restrict__ src, LimbAddr sa, u64 *__restrict__ dst, LimbAddr da, LimbMap map,
                                                 const PrimeConst *__restrict__ pc, NttTables tb, int logn, int inverse) {
    extern __shared__ u64 sm_dyn[];
    const int N = 1 << logn;
    const int li = blockIdx.x, pi = map.prime[li % map.n];
    const u64 q = pc[pi].q, q2 = q << 1;
    const u64 *p = src + sa.off(li, map.n, N);
    u64 *o = dst + da.off(li, map.n, N);
    for (int i = threadIdx.x; i < N; i += blockDim.x) sm_dyn[i] = p[i];
    __syncthreads();
    if (!inverse) {
        const u64 *w = tb.psi + (size_t)pi * N, *ws = tb.psi_sh + (size_t)pi * N;
        int t = N;
        for (int m = 1; m < N; m <<= 1) {
            t >>= 1;
            for (int k = threadIdx.x; k < N / 2; k += blockDim.x) {
                int i = k / t, j = k - i * t, i0 = 2 * i * t + j;
                ct_bfly(sm_dyn[i0], sm_dyn[i0 + t], w[m + i], ws[m + i], q, q2);
            }
            __syncthreads();
        }
        for (int i = threadIdx.x; i < N; i += blockDim.x) {
            u64 x = sm_dyn[i];
            x = x >= q2 ? x - q2 : x;
            o[i] = x >= q ? x - q : x;
        }
    } else {
        const u64 *w = tb.ipsi + (size_t)pi * N, *ws = tb.ipsi_sh + (size_t)pi * N;
        int t = 1;
        for (int m = N >> 1; m >= 1; m >>= 1) {
            for (int k = threadIdx.x; k < N / 2; k += blockDim.x) {
                int i = k / t, j = k - i * t, i0 = 2 * i * t + j;
                gs_bfly(sm_dyn[i0], sm_dyn[i0 + t], w[m + i], ws[m + i], q, q2);
            }
            __syncthreads();
            t <<= 1;
        }
        const u64 ninv = pc[pi].n_inv, ninv_sh = pc[pi].n_inv_sh;
        for (int i = threadIdx.x; i < N; i += blockDim.x) o[i] = mul_shoup(sm_dyn[i], ninv, ninv_sh, q);
    }
}

// Launch a batched transform of `count` limb instances.  src == dst gives an in-place transform;
// with distinct buffers `dst` also serves as the intermediate between the two passes.
inline cudaError_t launch_ntt(cudaStream_t st, const u64 *src, size_t src_outer, u64 *dst, size_t dst_outer, int count, const LimbMap &map,
                              const PrimeConst *pc, const NttTables &tb, int logn, bool inverse) {
    if (count == 0) return cudaSuccess;
    LimbAddr sa{src_outer}, da{dst_outer};
    if (logn == 16) {
        dim3 grid(16, count);
        if (!inverse) {
            ntt16_fwd_cols<<<grid, 256, 0, st>>>(src, sa, dst, da, map, pc, tb);
            ntt16_fwd_rows<<<grid, 256, 0, st>>>(dst, da, dst, da, map, pc, tb);
        } else {
            ntt16_inv_rows<<<grid, 256, 0, st>>>(src, sa, dst, da, map, pc, tb);
            ntt16_inv_cols<<<grid, 256, 0, st>>>(dst, da, dst, da, map, pc, tb);
        }
    } else if (logn <= 12) {
        ntt_small<<<count, 256, sizeof(u64) << logn, st>>>(src, sa, dst, da, map, pc, tb, logn, inverse ? 1 : 0);
    } else {
        return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

} // namespace hb
