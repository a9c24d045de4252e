// Negacyclic NTT / inverse NTT over RNS limbs for sm_100a: dispatch, and the small-degree kernel.
//
// Output order of the forward transform: a_hat[i] = a(psi^(2*bitrev(i)+1)); twiddle tables hold
// psi^bitrev(k) (forward) and psi^-bitrev(k) (inverse) with their Shoup companions.
//
// N = 2^16: the two-pass kernels of ntt16.cuh.
// N <= 4096 (small-parameter tests): one CTA transforms a whole limb in shared memory (below).
#pragma once
#include "modarith.cuh"
#include "ntt16.cuh"

namespace hb {

struct NttTables {
    const u64 *psi, *psi_sh, *ipsi, *ipsi_sh; // each [nprimes][N]: the small-degree kernel
    Ntt16Tables t16;                          // N = 2^16
};

// address of limb instance li: (li / map.n) * outer + (li % map.n) * N
struct LimbAddr {
    size_t outer;
    __device__ __forceinline__ size_t off(int li, int period, int N) const {
        return (size_t)(li / period) * outer + (size_t)(li % period) * N;
    }
};

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
                              const PrimeConst *pc, const NttTables &tb, int logn, bool inverse, const Ntt16Scale *scale = nullptr) {
    if (count == 0) return cudaSuccess;
    if (logn == 16) return launch_ntt16(st, src, src_outer, dst, dst_outer, count, map, pc, tb.t16, inverse, scale);
    if (scale) return cudaErrorInvalidValue; // only the 2^16 kernels take a scale
    if (logn > 12) return cudaErrorInvalidValue;
    LimbAddr sa{src_outer}, da{dst_outer};
    ntt_small<<<count, 256, sizeof(u64) << logn, st>>>(src, sa, dst, da, map, pc, tb, logn, inverse ? 1 : 0);
    return cudaGetLastError();
}

} // namespace hb
