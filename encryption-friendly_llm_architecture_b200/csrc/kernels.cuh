// Element-wise, base-conversion, automorphism, sampling and accumulate kernels (sm_100a).
// Arrays are dense [instances][N] uint64 unless a stride is named; instance li uses prime
// map.prime[li % map.n].  One thread handles one coefficient of one limb instance; a warp
// touches 256 contiguous bytes per array, so every stream is fully coalesced.  Gathers through
// ntt_perm stay inside an aligned 32-element block (the automorphism permutes aligned blocks
// of the bit-reversed index as units), so they cost no extra sectors.
#pragma once
#include "modarith.cuh"
#include "bulk.cuh"

namespace hb {

// Every thread handles kElems coefficients, blockDim apart (each access stays a 256-byte run per warp): four
// independent loads per array are in flight per thread and the grid has four times fewer, fatter CTAs --
// with one coefficient per thread these kernels were bound by CTA turnover at about 2 TB/s.
constexpr int kElems = 4;

// out = a + b  (mode 0) | a - b (mode 1) | -a (mode 2)
__global__ void k_addsub(u64 *__restrict__ out, const u64 *__restrict__ a, const u64 *__restrict__ b, LimbMap map, const PrimeConst *__restrict__ pc,
                         int N, int mode) {
    const int li = blockIdx.y;
#pragma unroll
    for (int u_ = 0; u_ < kElems; ++u_) {
        const int i = (blockIdx.x * kElems + u_) * blockDim.x + threadIdx.x;
        if (i >= N) break;
        const PrimeConst m = pc[map.prime[li % map.n]];
        const size_t off = (size_t)li * N + i;
        u64 x = a[off];
        if (mode == 0) out[off] = add_mod(x, b[off], m.q);
        else if (mode == 1) out[off] = sub_mod(x, b[off], m.q);
        else out[off] = x ? m.q - x : 0;
    }
}

struct Scalars { u64 v[kMaxPrimes]; };
// out = a * s[prime]
__global__ void k_scalar_mul(u64 *__restrict__ out, const u64 *__restrict__ a, size_t a_outer, LimbMap map, const PrimeConst *__restrict__ pc, int N, Scalars s) {
    const int li = blockIdx.y;
#pragma unroll
    for (int u_ = 0; u_ < kElems; ++u_) {
        const int i = (blockIdx.x * kElems + u_) * blockDim.x + threadIdx.x;
        if (i >= N) break;
        const int pi = map.prime[li % map.n];
        const PrimeConst m = pc[pi];
        const size_t soff = (size_t)(li / map.n) * a_outer + (size_t)(li % map.n) * N + i;
        out[(size_t)li * N + i] = mul_mod_any(a[soff], s.v[pi], m);
    }
}
// multiplication by X^(N/2): +iu on the first half of an NTT-form limb, -iu on the second
__global__ void k_mult_imag(u64 *__restrict__ out, const u64 *__restrict__ a, LimbMap map, const PrimeConst *__restrict__ pc, int N) {
    const int li = blockIdx.y;
#pragma unroll
    for (int u_ = 0; u_ < kElems; ++u_) {
        const int i = (blockIdx.x * kElems + u_) * blockDim.x + threadIdx.x;
        if (i >= N) break;
        const PrimeConst m = pc[map.prime[li % map.n]];
        const size_t off = (size_t)li * N + i;
        u64 r = mul_shoup(a[off], m.iu, m.iu_sh, m.q);
        if (i >= N / 2) r = r ? m.q - r : 0;
        out[off] = r;
    }
}
// out = a (.) pt, pt limb = li % map.n
__global__ void k_mul_pt(u64 *__restrict__ out, const u64 *__restrict__ a, const u64 *__restrict__ pt, LimbMap map, const PrimeConst *__restrict__ pc, int N) {
    const int li = blockIdx.y;
#pragma unroll
    for (int u_ = 0; u_ < kElems; ++u_) {
        const int i = (blockIdx.x * kElems + u_) * blockDim.x + threadIdx.x;
        if (i >= N) break;
        const PrimeConst m = pc[map.prime[li % map.n]];
        const size_t off = (size_t)li * N + i;
        out[off] = mul_mod_any(a[off], pt[(size_t)(li % map.n) * N + i], m);
    }
}
// out = a (.) pa + b (.) pb
__global__ void k_mul2_add(u64 *__restrict__ out, const u64 *__restrict__ a, const u64 *__restrict__ pa, const u64 *__restrict__ b, const u64 *__restrict__ pb,
                           LimbMap map, const PrimeConst *__restrict__ pc, int N) {
    const int li = blockIdx.y;
#pragma unroll
    for (int u_ = 0; u_ < kElems; ++u_) {
        const int i = (blockIdx.x * kElems + u_) * blockDim.x + threadIdx.x;
        if (i >= N) break;
        const PrimeConst m = pc[map.prime[li % map.n]];
        const size_t off = (size_t)li * N + i;
        const size_t po = (size_t)(li % map.n) * N + i;
        Acc128 s; s.zero();
        s.mad(a[off], pa[po]); s.mad(b[off], pb[po]);
        out[off] = barrett128(s.hi, s.lo, m);
    }
}
// tensor product, optional accumulation.  grid.y = batch * n; x, y: [groups][batch][2][n][N]; d: [batch][3][n][N]
//   d[b] (+)= sum over the groups g of tensor(x[g][b], y[g][b])
// (groups = 1 is the plain tensor product; several groups are several iterations of a product loop in one launch).
__global__ void k_tensor(u64 *__restrict__ d, const u64 *__restrict__ x, const u64 *__restrict__ y, int n, LimbMap map, const PrimeConst *__restrict__ pc, int N,
                         int accumulate, int groups, int batch) {
    const int bl = blockIdx.y, b = bl / n, l = bl % n;
    const size_t gstride = (size_t)batch * 2 * n * N;
#pragma unroll
    for (int u_ = 0; u_ < kElems; ++u_) {
        const int i = (blockIdx.x * kElems + u_) * blockDim.x + threadIdx.x;
        if (i >= N) break;
        const PrimeConst m = pc[map.prime[l]];
        const size_t x0 = ((size_t)(b * 2) * n + l) * N + i, x1 = x0 + (size_t)n * N;
        const size_t d0 = ((size_t)(b * 3) * n + l) * N + i, d1 = d0 + (size_t)n * N, d2 = d1 + (size_t)n * N;
        u64 r0, r1, r2;
        if (m.fp) { // lazy products below 1.6q; the group count is bounded by the launcher so that the sums stay below 2^52
            u64 s0 = 0, s1 = 0, s2 = 0;
            for (int g = 0; g < groups; ++g) {
                const u64 b1 = x[g * gstride + x0], a1 = x[g * gstride + x1], b2 = y[g * gstride + x0], a2 = y[g * gstride + x1];
                const double b1d = u52_to_double(b1), a1d = u52_to_double(a1), b2d = u52_to_double(b2), a2d = u52_to_double(a2);
                s0 += mul_small_lazy_d(b1, b1d, b2, b2d, m.q_inv_f, m.q);
                s2 += mul_small_lazy_d(a1, a1d, a2, a2d, m.q_inv_f, m.q);
                s1 += mul_small_lazy_d(a1, a1d, b2, b2d, m.q_inv_f, m.q) + mul_small_lazy_d(a2, a2d, b1, b1d, m.q_inv_f, m.q);
            }
            r0 = reduce_fp(s0, m.q_inv_f, m.q); r1 = reduce_fp(s1, m.q_inv_f, m.q); r2 = reduce_fp(s2, m.q_inv_f, m.q);
        } else {
            Acc128 s0, s1, s2; s0.zero(); s1.zero(); s2.zero();
            for (int g = 0; g < groups; ++g) {
                const u64 b1 = x[g * gstride + x0], a1 = x[g * gstride + x1], b2 = y[g * gstride + x0], a2 = y[g * gstride + x1];
                s0.mad(b1, b2); s2.mad(a1, a2); s1.mad(a1, b2); s1.mad(a2, b1);
            }
            r0 = barrett128(s0.hi, s0.lo, m); r1 = barrett128(s1.hi, s1.lo, m); r2 = barrett128(s2.hi, s2.lo, m);
        }
        if (accumulate) { r0 = add_mod(r0, d[d0], m.q); r1 = add_mod(r1, d[d1], m.q); r2 = add_mod(r2, d[d2], m.q); }
        d[d0] = r0; d[d1] = r1; d[d2] = r2;
    }
}
// out[li][i] = in[li][perm_g(i)]
__global__ void k_permute(u64 *__restrict__ out, const u64 *__restrict__ in, u32 g, int logn, int N) {
    const int li = blockIdx.y;
#pragma unroll
    for (int u_ = 0; u_ < kElems; ++u_) {
        const int i = (blockIdx.x * kElems + u_) * blockDim.x + threadIdx.x;
        if (i >= N) break;
        out[(size_t)li * N + i] = in[(size_t)li * N + ntt_perm((u32)i, g, logn)];
    }
}
// int64 coefficients -> residues of every limb instance (coefficient form)
__global__ void k_reduce_i64(u64 *__restrict__ out, const i64 *__restrict__ coef, LimbMap map, const PrimeConst *__restrict__ pc, int N) {
    const int li = blockIdx.y;
#pragma unroll
    for (int u_ = 0; u_ < kElems; ++u_) {
        const int i = (blockIdx.x * kElems + u_) * blockDim.x + threadIdx.x;
        if (i >= N) break;
        const PrimeConst m = pc[map.prime[li % map.n]];
        const size_t off = (size_t)li * N + i;
        out[off] = reduce_i64(coef[i], m);
    }
}
// x mod q for lazily summed residues
__global__ void k_mod_reduce(u64 *__restrict__ a, LimbMap map, const PrimeConst *__restrict__ pc, int N) {
    const int li = blockIdx.y;
#pragma unroll
    for (int u_ = 0; u_ < kElems; ++u_) {
        const int i = (blockIdx.x * kElems + u_) * blockDim.x + threadIdx.x;
        if (i >= N) break;
        const PrimeConst m = pc[map.prime[li % map.n]];
        const size_t off = (size_t)li * N + i;
        a[off] = reduce_u64(a[off], m);
    }
}
// out = (x_0 + ... + x_{count-1}) mod q for canonical residues (count <= 16: the sum stays below 2^64)
struct SumList { const u64 *x[16]; int count; };
__global__ void k_sum_mod(u64 *__restrict__ out, SumList sl, LimbMap map, const PrimeConst *__restrict__ pc, int N) {
    const int li = blockIdx.y;
#pragma unroll
    for (int u_ = 0; u_ < kElems; ++u_) {
        const int i = (blockIdx.x * kElems + u_) * blockDim.x + threadIdx.x;
        if (i >= N) break;
        const PrimeConst m = pc[map.prime[li % map.n]];
        const size_t off = (size_t)li * N + i;
        u64 v = 0;
        for (int t = 0; t < sl.count; ++t) v += sl.x[t][off];
        out[off] = reduce_u64(v, m);
    }
}

// ---------------- rescale ----------------
// t[bp][l][i] = centred(last[bp][i]) mod q_l, l < level.  grid.y = nbp * level
__global__ void k_rescale_prep(u64 *__restrict__ t, const u64 *__restrict__ last, int level, const PrimeConst *__restrict__ pc, int N) {
    const int w = blockIdx.y, bp = w / level, l = w % level;
#pragma unroll
    for (int u_ = 0; u_ < kElems; ++u_) {
        const int i = (blockIdx.x * kElems + u_) * blockDim.x + threadIdx.x;
        if (i >= N) break;
        const PrimeConst m = pc[l];
        const u64 ql = pc[level].q;
        const u64 r = last[(size_t)bp * N + i];
        const i64 centred = r > (ql >> 1) ? (i64)r - (i64)ql : (i64)r;
        t[(size_t)w * N + i] = reduce_i64_any(centred, m);
    }
}
// out[bp][l] = (x[bp][l] - t[bp][l]) * q_level^-1 ; x has level+1 limbs per poly
__global__ void k_rescale_fin(u64 *__restrict__ out, const u64 *__restrict__ x, const u64 *__restrict__ t, int level, const PrimeConst *__restrict__ pc, int N,
                              Scalars qlinv) {
    const int w = blockIdx.y, bp = w / level, l = w % level;
#pragma unroll
    for (int u_ = 0; u_ < kElems; ++u_) {
        const int i = (blockIdx.x * kElems + u_) * blockDim.x + threadIdx.x;
        if (i >= N) break;
        const PrimeConst m = pc[l];
        const u64 xv = x[((size_t)bp * (level + 1) + l) * N + i];
        out[(size_t)w * N + i] = mul_mod_any(sub_mod(xv, t[(size_t)w * N + i], m.q), qlinv.v[l], m);
    }
}

// ---------------- fused plaintext products with rescale ----------------
// out = sum_j rescale(a_j (.) p_j)          (separate == 1: every term is rescaled on its own, as
//                                             eval.mult(ct, mask) does, and the results are added)
// out = rescale(sum_j a_j (.) p_j)          (separate == 0: the "assemble" step)
// Rescale subtracts NTT_i(centred lift of the last limb) from limb i; NTT is linear modulo q_i, so the
// centred lifts of all terms are summed as integers first and ONE transform per limb serves the whole
// sum.  The stored residues equal those of the term-by-term sequence.
constexpr int kMaxTerms = 24;
struct TermList { const u64 *a[kMaxTerms]; const u64 *p[kMaxTerms]; int count; };
// last[g][bp][x] = (sum over the terms of group g) a_j[bp][level][x] * p_j[level][x] mod q_level
// grid = (N/256, nbp, groups)   groups = count (separate) or 1
__global__ void k_last_prod(u64 *__restrict__ last, TermList tl, int separate, int level, int nbp, const PrimeConst *__restrict__ pc, int N) {
#pragma unroll
    for (int u_ = 0; u_ < kElems; ++u_) {
        const int x = (blockIdx.x * kElems + u_) * blockDim.x + threadIdx.x;
        if (x >= N) break;
        const int bp = blockIdx.y, g = blockIdx.z;
        const PrimeConst m = pc[level];
        const size_t ao = ((size_t)bp * (level + 1) + level) * N + x, po = (size_t)level * N + x;
        const int j0 = separate ? g : 0, j1 = separate ? g + 1 : tl.count;
        u64 r;
        if (m.fp) {
            u64 acc = 0;
            for (int j = j0; j < j1; ++j) acc += mul_small_lazy(tl.a[j][ao], tl.p[j][po], m.q_inv_f, m.q);
            r = reduce_fp(acc, m.q_inv_f, m.q);
        } else {
            Acc128 s; s.zero();
            for (int j = j0; j < j1; ++j) s.mad(tl.a[j][ao], tl.p[j][po]);
            r = barrett128(s.hi, s.lo, m);
        }
        last[((size_t)g * nbp + bp) * N + x] = r;
    }
}
// S[bp][x] = sum_g centred(last[g][bp][x]) as a signed integer (|S| <= groups * q_level / 2)
__global__ void k_centre_sum(i64 *__restrict__ S, const u64 *__restrict__ last, int groups, int nbp, int level, const PrimeConst *__restrict__ pc, int N) {
#pragma unroll
    for (int u_ = 0; u_ < kElems; ++u_) {
        const int x = (blockIdx.x * kElems + u_) * blockDim.x + threadIdx.x;
        if (x >= N) break;
        const int bp = blockIdx.y;
        const u64 ql = pc[level].q, half = ql >> 1;
        i64 acc = 0;
        for (int g = 0; g < groups; ++g) {
            const u64 r = last[((size_t)g * nbp + bp) * N + x];
            acc += r > half ? (i64)r - (i64)ql : (i64)r;
        }
        S[(size_t)bp * N + x] = acc;
    }
}
// t[bp][l][x] = S[bp][x] mod q_l.  grid.y = nbp * level
__global__ void k_lift_mod(u64 *__restrict__ t, const i64 *__restrict__ S, int level, const PrimeConst *__restrict__ pc, int N) {
    const int w = blockIdx.y, bp = w / level, l = w % level;
#pragma unroll
    for (int u_ = 0; u_ < kElems; ++u_) {
        const int x = (blockIdx.x * kElems + u_) * blockDim.x + threadIdx.x;
        if (x >= N) break;
        t[(size_t)w * N + x] = reduce_i64_any(S[(size_t)bp * N + x], pc[l]);
    }
}
// out[bp][l][x] = (sum_j a_j[bp][l][x] * p_j[l][x] - t[bp][l][x]) * q_level^-1.  grid = (N/(256*kElems), nbp * level).
// The four coefficients of a thread sit in the inner loop so that eight loads of one term (and, unrolled, of the
// next) are in flight together: the kernel streams `count` ciphertexts per output and lives on memory parallelism.
// Blocks are ordered limb-major (all batch members of limb 0, then of limb 1, ...): the plaintext limbs of a sum are
// shared by every member, and in this order they stay in L2 while the members stream past.
__global__ void k_prod_rescale_fin(u64 *__restrict__ out, TermList tl, const u64 *__restrict__ t, int level, int nbp, const PrimeConst *__restrict__ pc, int N, Scalars qlinv) {
    const int l = blockIdx.y / nbp, bp = blockIdx.y % nbp, w = bp * level + l;
    const PrimeConst m = pc[l];
    const u32 x0 = blockIdx.x * (blockDim.x * kElems) + threadIdx.x;
    const size_t ao = ((size_t)bp * (level + 1) + l) * N + x0, po = (size_t)l * N + x0;
    u64 v[kElems];
    if (m.fp) {
        u64 acc[kElems];
#pragma unroll
        for (int u = 0; u < kElems; ++u) acc[u] = 0;
#pragma unroll 2
        for (int j = 0; j < tl.count; ++j) {
            const u64 *a = tl.a[j] + ao, *p = tl.p[j] + po;
#pragma unroll
            for (int u = 0; u < kElems; ++u) acc[u] += mul_small_lazy(a[u * blockDim.x], p[u * blockDim.x], m.q_inv_f, m.q);
        }
#pragma unroll
        for (int u = 0; u < kElems; ++u) v[u] = reduce_fp(acc[u], m.q_inv_f, m.q);
    } else {
        Acc128 s[kElems];
#pragma unroll
        for (int u = 0; u < kElems; ++u) s[u].zero();
#pragma unroll 2
        for (int j = 0; j < tl.count; ++j) {
            const u64 *a = tl.a[j] + ao, *p = tl.p[j] + po;
#pragma unroll
            for (int u = 0; u < kElems; ++u) s[u].mad(a[u * blockDim.x], p[u * blockDim.x]);
        }
#pragma unroll
        for (int u = 0; u < kElems; ++u) v[u] = barrett128(s[u].hi, s[u].lo, m);
    }
    const u64 *tp = t + (size_t)w * N + x0;
    u64 *op = out + (size_t)w * N + x0;
#pragma unroll
    for (int u = 0; u < kElems; ++u) op[u * blockDim.x] = mul_mod_any(sub_mod(v[u], tp[u * blockDim.x], m.q), qlinv.v[l], m);
}

// ---- the same for all giant-step parts of a baby-step / giant-step transform at once ----
// A transform with bs baby rotations a_j and 2 gs parts computes  out_g = rescale(sum_j a_j (.) p_gj): every part reads
// the same a_j.  One pass per limb keeps a part accumulator per g in registers and reads every a_j once (and, for
// primes below 2^44, converts it once) instead of once per part; the masks p_gj are shared by all members and come
// from L2.  Absent terms of a part are null pointers.
constexpr int kMaxParts = 17, kMaxPartTerms = 17;
struct PartTerms { const u64 *a[kMaxPartTerms]; const u64 *p[kMaxParts][kMaxPartTerms]; int count, parts; };
// A CTA of 1024 threads keeps the mask chunks of G parts for its 256 coefficients of one limb in shared memory (bulk
// copies, up to G * 17 chunks of 2 KB, one mbarrier, bounded wait) and walks over the batch members, four at a time
// (thread = coefficient + 256 * member slot): the masks cross L2 once per CTA instead of once per member, the a_j of a
// member are read by the ceil(parts / G) CTAs of the chunk (from L2 after the first), and every thread has the next
// two a_j in flight while it works on the current one.
// t == nullptr: raw sums of limb `level`, out[(g * nbp + bp) * N + x]                       grid = (N/256, 1, ceil(parts/G))
// else: out[((g * nbp + bp) * level + l) * N + x] = (sum - t[same]) * q_level^-1 mod q_l      grid = (N/256, level, ceil(parts/G))
template <int G>
__global__ void __launch_bounds__(1024, 1) k_prod_parts(u64 *__restrict__ out, const __grid_constant__ PartTerms pt, const u64 *__restrict__ t, int level, int nbp,
                                                        const PrimeConst *__restrict__ pc, int N, const __grid_constant__ Scalars qlinv, int *__restrict__ err) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ __align__(8) u64 bar;
    u64 *ptile = reinterpret_cast<u64 *>(smem_raw); // [G][count][256]
    const int tid = threadIdx.x, lane = tid & 255, slot = tid >> 8;
    const int l = t ? (int)blockIdx.y : level, g0 = blockIdx.z * G, count = pt.count;
    const int gn = min(G, pt.parts - g0);
    const u32 x0 = blockIdx.x * 256;
    if (tid == 0) { mbar_init(&bar, 1); mbar_fence_init(); }
    __syncthreads();
    if (tid < 32) {
        if (tid == 0) {
            u32 present = 0;
            for (int ci = 0; ci < gn * count; ++ci) present += pt.p[g0 + ci / count][ci % count] != nullptr;
            mbar_arrive_expect_tx(&bar, present * 2048u);
        }
        __syncwarp();
        for (int ci = tid; ci < gn * count; ci += 32) {
            const u64 *src = pt.p[g0 + ci / count][ci % count];
            if (src) bulk_load(ptile + (size_t)ci * 256, src + (size_t)l * N + x0, 2048u, &bar);
        }
    }
    u32 have[G]; // bit j: part g0 + g has term j
#pragma unroll
    for (int g = 0; g < G; ++g) {
        have[g] = 0;
        if (g < gn)
            for (int j = 0; j < count; ++j) have[g] |= (pt.p[g0 + g][j] != nullptr ? 1u : 0u) << j;
    }
    mbar_wait_bounded(&bar, 0, err);
    const PrimeConst m = pc[l];
    const u64 qli = t ? qlinv.v[l] : 0;
    const double qd = (double)m.q;
    // Absent terms get zero masks, so the product loop below is straight-line code (no test per part and term: the
    // independent chains of the G parts interleave); the masks of a prime below 2^44 become doubles once.
#pragma unroll
    for (int g = 0; g < G; ++g)
        for (int j = slot; j < count; j += 4) {
            u64 *w = ptile + (size_t)(g * count + j) * 256 + lane;
            if (!((have[g] >> j) & 1u)) *w = 0;
            else if (m.fp) *w = (u64)__double_as_longlong(u52_to_double(*w));
        }
    __syncthreads();
    for (int bp = slot; bp < nbp; bp += 4) {
        const size_t ao = ((size_t)bp * (level + 1) + l) * N + x0 + lane;
        u64 v[G];
        u64 a_cur = pt.a[0][ao], a_nxt = count > 1 ? pt.a[1][ao] : 0;
        if (m.fp) { // products entirely on the FP64 pipe, signed double sums (17 terms of at most 0.51 q each)
            double acc[G];
#pragma unroll
            for (int g = 0; g < G; ++g) acc[g] = 0.0;
            const double *dtile = reinterpret_cast<const double *>(ptile);
            for (int j = 0; j < count; ++j) {
                const u64 a = a_cur;
                a_cur = a_nxt;
                if (j + 2 < count) a_nxt = pt.a[j + 2][ao];
                const double ad = u52_to_double(a);
#pragma unroll
                for (int g = 0; g < G; ++g) acc[g] = __dadd_rn(acc[g], mul_fp64_lazy(ad, dtile[(size_t)(g * count + j) * 256 + lane], m.q_inv_f, qd));
            }
#pragma unroll
            for (int g = 0; g < G; ++g) v[g] = canon_fp64(acc[g], m.q_inv_f, qd);
        } else {
            Acc128 acc[G];
#pragma unroll
            for (int g = 0; g < G; ++g) acc[g].zero();
            for (int j = 0; j < count; ++j) {
                const u64 a = a_cur;
                a_cur = a_nxt;
                if (j + 2 < count) a_nxt = pt.a[j + 2][ao];
#pragma unroll
                for (int g = 0; g < G; ++g) acc[g].mad(a, ptile[(size_t)(g * count + j) * 256 + lane]);
            }
#pragma unroll
            for (int g = 0; g < G; ++g) v[g] = barrett128(acc[g].hi, acc[g].lo, m);
        }
#pragma unroll
        for (int g = 0; g < G; ++g)
            if (g < gn) {
                if (t) {
                    const size_t w = (((size_t)(g0 + g) * nbp + bp) * level + l) * N + x0 + lane;
                    out[w] = mul_mod_any(sub_mod(v[g], t[w], m.q), qli, m);
                } else out[((size_t)(g0 + g) * nbp + bp) * N + x0 + lane] = v[g];
            }
    }
}

// ---------------- key switching ----------------
// Per-level plan held in device memory.
struct KsPlan {
    int level, n, ne, nd, K;
    int dt_count;                               // lifted (non-own) limbs over all digits
    int dig_lo[8], dig_hi[8];                   // own limb range of each digit
    int dt_start[8];                            // first compact entry of each digit
    short dt_entry[8][kMaxPrimes];              // [digit][ext limb j] -> compact entry or -1 (own)
    unsigned char ext_prime[kMaxPrimes];        // ext limb j -> prime index
    u64 hat_inv[8][kMaxDigitLimbs], hat_inv_sh[8][kMaxDigitLimbs];
    u64 hat_mod[8][kMaxDigitLimbs][kMaxPrimes]; // [digit][source][ext limb j]
    u64 hat_mod_d0[8][kMaxDigitLimbs][kMaxPrimes]; // the same as a double (bit pattern), and times 2^30 mod the target: for
    u64 hat_mod_d1[8][kMaxDigitLimbs][kMaxPrimes]; // targets below 2^44 the conversion runs on the FP64 pipe
    u64 p_hat_inv[8], p_hat_inv_sh[8];          // ModDown: per special prime
    u64 p_hat_mod[8][kMaxPrimes];               // [special k][q limb l]
    u64 p_hat_mod_d0[8][kMaxPrimes], p_hat_mod_d1[8][kMaxPrimes]; // as doubles, and times 2^30 mod q_l
    u64 p_inv[kMaxPrimes];                      // P^-1 mod q_l
};

// ModUp: a_coef [batch][n][N] (coefficient form) -> dt [batch][dt_count][N] (coefficient form).
// grid = (N/256, nd, batch).  The source count of a digit is a template parameter so that the per-target
// contraction is fully unrolled with no predicated-off iterations.
template <int NS>
__device__ __forceinline__ void modup_body(u64 *__restrict__ dt, const u64 *__restrict__ a_coef, const KsPlan *__restrict__ pl, const PrimeConst *__restrict__ pc, int N,
                                           int i, int dg, int b) {
    const int lo = pl->dig_lo[dg], hi = lo + NS, n = pl->n, ne = pl->ne;
    u64 y[NS];
#pragma unroll
    for (int s = 0; s < NS; ++s) y[s] = mul_shoup(a_coef[((size_t)b * n + lo + s) * N + i], pl->hat_inv[dg][s], pl->hat_inv_sh[dg][s], pc[lo + s].q);
    u64 *o = dt + ((size_t)b * pl->dt_count + pl->dt_start[dg]) * N + i;
    double y0[NS], y1[NS]; // 30-bit pieces of the sources as doubles, for the targets below 2^44
#pragma unroll
    for (int k = 0; k < NS; ++k) {
        y0[k] = __hiloint2double(0x43300000, (int)((u32)y[k] & 0x3FFFFFFFu)) - kTwo52;
        y1[k] = __hiloint2double(0x43300000, (int)(u32)(y[k] >> 30)) - kTwo52;
    }
    for (int j = 0; j < ne; ++j) {
        if (j >= lo && j < hi) continue;
        const PrimeConst *m = pc + pl->ext_prime[j];
        if (m->fp) {
            const double qinv = m->q_inv_f, qd = (double)m->q;
            double acc = 0.0;
#pragma unroll
            for (int k = 0; k < NS; ++k) {
                acc = __dadd_rn(acc, mul_fp64_lazy(y0[k], __longlong_as_double((long long)pl->hat_mod_d0[dg][k][j]), qinv, qd));
                acc = __dadd_rn(acc, mul_fp64_lazy(y1[k], __longlong_as_double((long long)pl->hat_mod_d1[dg][k][j]), qinv, qd));
            }
            *o = canon_fp64(acc, qinv, qd);
        } else {
            PieceAcc s; s.zero(); // at most 8 sources
#pragma unroll
            for (int k = 0; k < NS; ++k) s.mac(y[k], pl->hat_mod[dg][k][j]);
            PrimeConst mm; mm.q = m->q; mm.mu_hi = m->mu_hi; mm.mu_lo = m->mu_lo;
            *o = s.finish(mm);
        }
        o += N;
    }
}
__global__ void k_modup(u64 *__restrict__ dt, const u64 *__restrict__ a_coef, const KsPlan *__restrict__ pl, const PrimeConst *__restrict__ pc, int N) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= N) return;
    const int dg = blockIdx.y, b = blockIdx.z;
    switch (pl->dig_hi[dg] - pl->dig_lo[dg]) {
    case 1: modup_body<1>(dt, a_coef, pl, pc, N, i, dg, b); break;
    case 2: modup_body<2>(dt, a_coef, pl, pc, N, i, dg, b); break;
    case 3: modup_body<3>(dt, a_coef, pl, pc, N, i, dg, b); break;
    case 4: modup_body<4>(dt, a_coef, pl, pc, N, i, dg, b); break;
    case 5: modup_body<5>(dt, a_coef, pl, pc, N, i, dg, b); break;
    case 6: modup_body<6>(dt, a_coef, pl, pc, N, i, dg, b); break;
    case 7: modup_body<7>(dt, a_coef, pl, pc, N, i, dg, b); break;
    default: modup_body<8>(dt, a_coef, pl, pc, N, i, dg, b); break;
    }
}

// Inner product with the switching key over Q_level u P.
//   acc[b][p][j][i] = sum_dg digit_dg[j][perm_g(i)] * key[dg][p][prime(j)][i]
// digit_dg[j] is a_ntt[j] for own limbs and dt[...] otherwise.  grid = (N/(256*kElems), batch, ne)
__global__ void k_ks_inner(u64 *__restrict__ acc, const u64 *__restrict__ a_ntt, size_t a_outer, const u64 *__restrict__ dt, const u64 *__restrict__ key, int key_primes,
                           const KsPlan *__restrict__ pl, const PrimeConst *__restrict__ pc, u32 g, int logn, int N) {
    const int j = blockIdx.z, b = blockIdx.y; // limb-major block order: the key limbs stay in L2 across the members
    const int pj = pl->ext_prime[j], nd = pl->nd, ne = pl->ne;
    const PrimeConst m = pc[pj];
    const u32 x0 = blockIdx.x * (blockDim.x * kElems) + threadIdx.x;
    u32 src[kElems];
#pragma unroll
    for (int u = 0; u < kElems; ++u) { const u32 i = x0 + u * blockDim.x; src[u] = g ? ntt_perm(i, g, logn) : i; }
    const u64 *abase = a_ntt + (size_t)b * a_outer + (size_t)j * N;
    const u64 *dbase = dt + (size_t)b * pl->dt_count * N;
    const u64 *kbase = key + (size_t)pj * N + x0;
    const size_t kpoly = (size_t)key_primes * N;
    u64 r0[kElems], r1[kElems];
    if (m.fp) { // products on the FP64 pipe, signed double sums
        const double qd = (double)m.q;
        double d0[kElems], d1[kElems];
#pragma unroll
        for (int u = 0; u < kElems; ++u) { d0[u] = 0.0; d1[u] = 0.0; }
        for (int dg = 0; dg < nd; ++dg) {
            const int en = pl->dt_entry[dg][j];
            const u64 *sp = en < 0 ? abase : dbase + (size_t)en * N;
            const u64 *k0 = kbase + (size_t)dg * 2 * kpoly;
#pragma unroll
            for (int u = 0; u < kElems; ++u) {
                const double vd = u52_to_double(sp[src[u]]);
                d0[u] = __dadd_rn(d0[u], mul_fp64_lazy(vd, u52_to_double(k0[u * blockDim.x]), m.q_inv_f, qd));
                d1[u] = __dadd_rn(d1[u], mul_fp64_lazy(vd, u52_to_double(k0[kpoly + u * blockDim.x]), m.q_inv_f, qd));
            }
        }
#pragma unroll
        for (int u = 0; u < kElems; ++u) { r0[u] = canon_fp64(d0[u], m.q_inv_f, qd); r1[u] = canon_fp64(d1[u], m.q_inv_f, qd); }
    } else {
        Acc128 s0[kElems], s1[kElems];
#pragma unroll
        for (int u = 0; u < kElems; ++u) { s0[u].zero(); s1[u].zero(); }
        for (int dg = 0; dg < nd; ++dg) {
            const int en = pl->dt_entry[dg][j];
            const u64 *sp = en < 0 ? abase : dbase + (size_t)en * N;
            const u64 *k0 = kbase + (size_t)dg * 2 * kpoly;
#pragma unroll
            for (int u = 0; u < kElems; ++u) {
                const u64 v = sp[src[u]];
                s0[u].mad(v, k0[u * blockDim.x]);
                s1[u].mad(v, k0[kpoly + u * blockDim.x]);
            }
        }
#pragma unroll
        for (int u = 0; u < kElems; ++u) { r0[u] = barrett128(s0[u].hi, s0[u].lo, m); r1[u] = barrett128(s1[u].hi, s1[u].lo, m); }
    }
    u64 *o0 = acc + (((size_t)b * 2) * ne + j) * N + x0, *o1 = o0 + (size_t)ne * N;
#pragma unroll
    for (int u = 0; u < kElems; ++u) { o0[u * blockDim.x] = r0[u]; o1[u * blockDim.x] = r1[u]; }
}

// ModDown conversion: pcoef [bp][K][N] (special limbs, coefficient form) -> t [bp][n][N] (coefficient form)
// grid = (N/256, 1, nbp)
template <int K>
__device__ __forceinline__ void moddown_conv_body(u64 *__restrict__ t, const u64 *__restrict__ pcoef, const KsPlan *__restrict__ pl, const PrimeConst *__restrict__ pc, int Lp1,
                                                  int N, int i, int bp) {
    const int n = pl->n;
    u64 y[K];
#pragma unroll
    for (int k = 0; k < K; ++k) y[k] = mul_shoup(pcoef[((size_t)bp * K + k) * N + i], pl->p_hat_inv[k], pl->p_hat_inv_sh[k], pc[Lp1 + k].q);
    u64 *o = t + (size_t)bp * n * N + i;
    double y0[K], y1[K]; // 30-bit pieces of the sources as doubles, for the targets below 2^44
#pragma unroll
    for (int k = 0; k < K; ++k) {
        y0[k] = __hiloint2double(0x43300000, (int)((u32)y[k] & 0x3FFFFFFFu)) - kTwo52;
        y1[k] = __hiloint2double(0x43300000, (int)(u32)(y[k] >> 30)) - kTwo52;
    }
    for (int l = 0; l < n; ++l) {
        if (pc[l].fp) {
            const double qinv = pc[l].q_inv_f, qd = (double)pc[l].q;
            double acc = 0.0;
#pragma unroll
            for (int k = 0; k < K; ++k) {
                acc = __dadd_rn(acc, mul_fp64_lazy(y0[k], __longlong_as_double((long long)pl->p_hat_mod_d0[k][l]), qinv, qd));
                acc = __dadd_rn(acc, mul_fp64_lazy(y1[k], __longlong_as_double((long long)pl->p_hat_mod_d1[k][l]), qinv, qd));
            }
            *o = canon_fp64(acc, qinv, qd);
        } else {
            PieceAcc s; s.zero();
#pragma unroll
            for (int k = 0; k < K; ++k) s.mac(y[k], pl->p_hat_mod[k][l]);
            PrimeConst mm; mm.q = pc[l].q; mm.mu_hi = pc[l].mu_hi; mm.mu_lo = pc[l].mu_lo;
            *o = s.finish(mm);
        }
        o += N;
    }
}
__global__ void k_moddown_conv(u64 *__restrict__ t, const u64 *__restrict__ pcoef, const KsPlan *__restrict__ pl, const PrimeConst *__restrict__ pc, int Lp1, int N) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= N) return;
    const int bp = blockIdx.z;
    switch (pl->K) {
    case 1: moddown_conv_body<1>(t, pcoef, pl, pc, Lp1, N, i, bp); break;
    case 2: moddown_conv_body<2>(t, pcoef, pl, pc, Lp1, N, i, bp); break;
    case 3: moddown_conv_body<3>(t, pcoef, pl, pc, Lp1, N, i, bp); break;
    case 4: moddown_conv_body<4>(t, pcoef, pl, pc, Lp1, N, i, bp); break;
    case 5: moddown_conv_body<5>(t, pcoef, pl, pc, Lp1, N, i, bp); break;
    case 6: moddown_conv_body<6>(t, pcoef, pl, pc, Lp1, N, i, bp); break;
    case 7: moddown_conv_body<7>(t, pcoef, pl, pc, Lp1, N, i, bp); break;
    default: moddown_conv_body<8>(t, pcoef, pl, pc, Lp1, N, i, bp); break;
    }
}
// out[b][p][l][i] = (acc[b][p][l][i] - t[b][p][l][i]) * P^-1 + add_p[b][l][perm_g(i)]
// add0 / add1 may be null; perm applies when g != 0.  grid = (N/256, n, batch*2)
__global__ void k_moddown_fin(u64 *__restrict__ out, size_t out_outer, const u64 *__restrict__ acc, const u64 *__restrict__ t, const u64 *__restrict__ add0,
                              const u64 *__restrict__ add1, size_t add_outer, const KsPlan *__restrict__ pl, const PrimeConst *__restrict__ pc, u32 g, int logn, int N) {
#pragma unroll
    for (int u_ = 0; u_ < kElems; ++u_) {
        const int i = (blockIdx.x * kElems + u_) * blockDim.x + threadIdx.x;
        if (i >= N) break;
        const int l = blockIdx.y, bp = blockIdx.z, b = bp >> 1, p = bp & 1;
        const int n = pl->n, ne = pl->ne;
        const PrimeConst m = pc[l];
        u64 v = sub_mod(acc[((size_t)bp * ne + l) * N + i], t[((size_t)bp * n + l) * N + i], m.q);
        v = mul_mod_any(v, pl->p_inv[l], m);
        const u64 *ad = p ? add1 : add0;
        if (ad) {
            const u32 s = g ? ntt_perm((u32)i, g, logn) : (u32)i;
            v = add_mod(v, ad[(size_t)b * add_outer + (size_t)l * N + s], m.q);
        }
        out[(size_t)b * out_outer + ((size_t)p * n + l) * N + i] = v;
    }
}

// ---------------- sum of rotations with one ModDown ----------------
// Up to 16 terms (ciphertext batch x_t rotated by g_t): the inner products of all terms are added up in Q_level u P.
struct RotTerm { const u64 *a_ntt; const u64 *dt; const u64 *key; u32 g; u32 pad; };
struct RotTermList { RotTerm t[16]; int count; };
//   acc[b][p][j][i] = sum_t sum_dg digit_t,dg[j][perm_t(i)] * key_t[dg][p][prime(j)][i]      grid = (N/(256*kElems), batch, ne)
__global__ void k_ks_inner_sum(u64 *__restrict__ acc, RotTermList tl, size_t a_outer, int key_primes, const KsPlan *__restrict__ pl, const PrimeConst *__restrict__ pc,
                               int logn, int N) {
    const int j = blockIdx.z, b = blockIdx.y;
    const int pj = pl->ext_prime[j], nd = pl->nd, ne = pl->ne;
    const PrimeConst m = pc[pj];
    const u32 x0 = blockIdx.x * (blockDim.x * kElems) + threadIdx.x;
    const size_t kpoly = (size_t)key_primes * N;
    u64 r0[kElems], r1[kElems];
    if (m.fp) { // at most 16 terms x 8 digits of products within 0.51 q of zero: signed double sums far below 2^53
        const double qd = (double)m.q;
        double d0[kElems], d1[kElems];
#pragma unroll
        for (int u = 0; u < kElems; ++u) { d0[u] = 0.0; d1[u] = 0.0; }
        for (int t = 0; t < tl.count; ++t) {
            u32 src[kElems];
#pragma unroll
            for (int u = 0; u < kElems; ++u) src[u] = ntt_perm(x0 + u * blockDim.x, tl.t[t].g, logn);
            const u64 *abase = tl.t[t].a_ntt + (size_t)b * a_outer + (size_t)j * N;
            const u64 *dbase = tl.t[t].dt + (size_t)b * pl->dt_count * N;
            const u64 *kbase = tl.t[t].key + (size_t)pj * N + x0;
            for (int dg = 0; dg < nd; ++dg) {
                const int en = pl->dt_entry[dg][j];
                const u64 *sp = en < 0 ? abase : dbase + (size_t)en * N;
                const u64 *k0 = kbase + (size_t)dg * 2 * kpoly;
#pragma unroll
                for (int u = 0; u < kElems; ++u) {
                    const double vd = u52_to_double(sp[src[u]]);
                    d0[u] = __dadd_rn(d0[u], mul_fp64_lazy(vd, u52_to_double(k0[u * blockDim.x]), m.q_inv_f, qd));
                    d1[u] = __dadd_rn(d1[u], mul_fp64_lazy(vd, u52_to_double(k0[kpoly + u * blockDim.x]), m.q_inv_f, qd));
                }
            }
        }
#pragma unroll
        for (int u = 0; u < kElems; ++u) { r0[u] = canon_fp64(d0[u], m.q_inv_f, qd); r1[u] = canon_fp64(d1[u], m.q_inv_f, qd); }
    } else {   // 64 products below 2^120 fit the 128-bit accumulator
        Acc128 s0[kElems], s1[kElems];
#pragma unroll
        for (int u = 0; u < kElems; ++u) { s0[u].zero(); s1[u].zero(); }
        for (int t = 0; t < tl.count; ++t) {
            u32 src[kElems];
#pragma unroll
            for (int u = 0; u < kElems; ++u) src[u] = ntt_perm(x0 + u * blockDim.x, tl.t[t].g, logn);
            const u64 *abase = tl.t[t].a_ntt + (size_t)b * a_outer + (size_t)j * N;
            const u64 *dbase = tl.t[t].dt + (size_t)b * pl->dt_count * N;
            const u64 *kbase = tl.t[t].key + (size_t)pj * N + x0;
            for (int dg = 0; dg < nd; ++dg) {
                const int en = pl->dt_entry[dg][j];
                const u64 *sp = en < 0 ? abase : dbase + (size_t)en * N;
                const u64 *k0 = kbase + (size_t)dg * 2 * kpoly;
#pragma unroll
                for (int u = 0; u < kElems; ++u) {
                    const u64 v = sp[src[u]];
                    s0[u].mad(v, k0[u * blockDim.x]);
                    s1[u].mad(v, k0[kpoly + u * blockDim.x]);
                }
            }
        }
#pragma unroll
        for (int u = 0; u < kElems; ++u) { r0[u] = barrett128(s0[u].hi, s0[u].lo, m); r1[u] = barrett128(s1[u].hi, s1[u].lo, m); }
    }
    u64 *o0 = acc + (((size_t)b * 2) * ne + j) * N + x0, *o1 = o0 + (size_t)ne * N;
#pragma unroll
    for (int u = 0; u < kElems; ++u) { o0[u * blockDim.x] = r0[u]; o1[u * blockDim.x] = r1[u]; }
}
// add[b][p][l][i] = sum over the rotated terms of (p == 0) c0_t[b][l][perm_t(i)]  +  sum over the unrotated terms of x_t[b][p][l][i]
// rot: terms with g != 1 (a_ntt - n limbs = c0); plain: terms added as they are.  grid = (N/(256*kElems), n, batch*2)
struct PlainTermList { const u64 *x[16]; int count; };
__global__ void k_rot_sum_addend(u64 *__restrict__ add, RotTermList rot, PlainTermList plain, int n, LimbMap map, const PrimeConst *__restrict__ pc, int logn, int N) {
    const int l = blockIdx.y, bp = blockIdx.z, b = bp >> 1, p = bp & 1;
    const u64 q = pc[map.prime[l]].q;
    const size_t ct_outer = (size_t)2 * n * N;
#pragma unroll
    for (int u_ = 0; u_ < kElems; ++u_) {
        const int i = (blockIdx.x * kElems + u_) * blockDim.x + threadIdx.x;
        if (i >= N) break;
        u64 v = 0;
        if (p == 0)
            for (int t = 0; t < rot.count; ++t) // a_ntt points at the second polynomial; the first sits n limbs before it
                v = add_mod(v, (rot.t[t].a_ntt - (size_t)n * N)[(size_t)b * ct_outer + (size_t)l * N + ntt_perm((u32)i, rot.t[t].g, logn)], q);
        for (int t = 0; t < plain.count; ++t) v = add_mod(v, plain.x[t][(size_t)b * ct_outer + ((size_t)p * n + l) * N + i], q);
        add[((size_t)bp * n + l) * N + i] = v;
    }
}

// ---------------- masked pair of rotations with one division by P * q_level ----------------
// Constants of the division of a Q_level u P polynomial by D = P * q_level (sources: q_level, p_1 .. p_K).
struct DivPlan {
    int level, ns;                     // ns = K + 1 source limbs
    unsigned char src_prime[8];
    u64 hat_inv[8], hat_inv_sh[8];     // (D / d_s)^-1 mod d_s
    u64 hat_mod[8][kMaxPrimes];        // (D / d_s) mod q_i, i < level
    u64 hat_mod_d0[8][kMaxPrimes];     // the same as a double (bit pattern), for targets below 2^44
    u64 hat_mod_d1[8][kMaxPrimes];     // (D / d_s) * 2^30 mod q_i as a double (bit pattern)
    u64 d_inv[kMaxPrimes];             // D^-1 mod q_i
    u64 p_mod[kMaxPrimes];             // P mod q_j, j <= level
};
struct RotPair {                       // the two rotations of one call
    const u64 *key[2];                 // switching keys
    const u64 *mask[2];                // extended plaintexts [ne][N]
    u32 g[2];
};
// E[b][p][j][i] = sum_r mask_r[j][i] * (sum_dg digit_dg[j][perm_r(i)] * key_r[dg][p][prime(j)][i])
//               + (p == 0 and j < n)  P * sum_r mask_r[j][i] * c0[b][j][perm_r(i)]
// Every term is reduced to its canonical residue before the next operation uses it.  grid = (N/(256*kElems), ne, batch)
__global__ void k_ks_inner_pair(u64 *__restrict__ E, const u64 *__restrict__ c0, const u64 *__restrict__ a_ntt, size_t a_outer, const u64 *__restrict__ dt, RotPair rp,
                                int key_primes, const KsPlan *__restrict__ pl, const DivPlan *__restrict__ dv, const PrimeConst *__restrict__ pc, int logn, int N) {
    const int j = blockIdx.y, b = blockIdx.z;
    const int pj = pl->ext_prime[j], nd = pl->nd, ne = pl->ne, n = pl->n;
    const PrimeConst m = pc[pj];
    const u32 x0 = blockIdx.x * (blockDim.x * kElems) + threadIdx.x;
    const u64 *abase = a_ntt + (size_t)b * a_outer + (size_t)j * N;
    const u64 *cbase = c0 + (size_t)b * a_outer + (size_t)j * N;
    const u64 *dbase = dt + (size_t)b * pl->dt_count * N;
    const size_t kpoly = (size_t)key_primes * N;
    u64 e0[kElems], e1[kElems], f[kElems];
#pragma unroll
    for (int u = 0; u < kElems; ++u) { e0[u] = 0; e1[u] = 0; f[u] = 0; }
    // When both steps are the same rotation (a row shift by a whole tile height on a full slot grid) the two inner
    // products are the same polynomial: it is computed once and multiplied by mask_0 + mask_1, which gives the same
    // residues as the two-term sum.
    const int nrot = rp.g[0] == rp.g[1] ? 1 : 2;
    for (int r = 0; r < nrot; ++r) {
        u32 src[kElems];
#pragma unroll
        for (int u = 0; u < kElems; ++u) src[u] = ntt_perm(x0 + u * blockDim.x, rp.g[r], logn);
        const u64 *kbase = rp.key[r] + (size_t)pj * N + x0;
        u64 r0[kElems], r1[kElems];
        if (m.fp) {
#pragma unroll
            for (int u = 0; u < kElems; ++u) { r0[u] = 0; r1[u] = 0; }
            for (int dg = 0; dg < nd; ++dg) {
                const int en = pl->dt_entry[dg][j];
                const u64 *sp = en < 0 ? abase : dbase + (size_t)en * N;
                const u64 *k0 = kbase + (size_t)dg * 2 * kpoly;
#pragma unroll
                for (int u = 0; u < kElems; ++u) {
                    const u64 v = sp[src[u]], ka = k0[u * blockDim.x], kb = k0[kpoly + u * blockDim.x];
                    const double vd = u52_to_double(v);
                    r0[u] += mul_small_lazy_d(v, vd, ka, u52_to_double(ka), m.q_inv_f, m.q);
                    r1[u] += mul_small_lazy_d(v, vd, kb, u52_to_double(kb), m.q_inv_f, m.q);
                }
            }
#pragma unroll
            for (int u = 0; u < kElems; ++u) { r0[u] = reduce_fp(r0[u], m.q_inv_f, m.q); r1[u] = reduce_fp(r1[u], m.q_inv_f, m.q); }
        } else {
            Acc128 s0[kElems], s1[kElems];
#pragma unroll
            for (int u = 0; u < kElems; ++u) { s0[u].zero(); s1[u].zero(); }
            for (int dg = 0; dg < nd; ++dg) {
                const int en = pl->dt_entry[dg][j];
                const u64 *sp = en < 0 ? abase : dbase + (size_t)en * N;
                const u64 *k0 = kbase + (size_t)dg * 2 * kpoly;
#pragma unroll
                for (int u = 0; u < kElems; ++u) {
                    const u64 v = sp[src[u]];
                    s0[u].mad(v, k0[u * blockDim.x]);
                    s1[u].mad(v, k0[kpoly + u * blockDim.x]);
                }
            }
#pragma unroll
            for (int u = 0; u < kElems; ++u) { r0[u] = barrett128(s0[u].hi, s0[u].lo, m); r1[u] = barrett128(s1[u].hi, s1[u].lo, m); }
        }
        const u64 *mk = rp.mask[r] + (size_t)j * N + x0, *mk2 = rp.mask[1] + (size_t)j * N + x0;
#pragma unroll
        for (int u = 0; u < kElems; ++u) {
            u64 w = mk[u * blockDim.x];
            if (nrot == 1) w = add_mod(w, mk2[u * blockDim.x], m.q);
            e0[u] = add_mod(e0[u], mul_mod_any(w, r0[u], m), m.q);
            e1[u] = add_mod(e1[u], mul_mod_any(w, r1[u], m), m.q);
            if (j < n) f[u] = add_mod(f[u], mul_mod_any(w, cbase[src[u]], m), m.q);
        }
    }
    if (j < n) {
        const u64 pm = dv->p_mod[j];
#pragma unroll
        for (int u = 0; u < kElems; ++u) e0[u] = add_mod(e0[u], mul_mod_any(pm, f[u], m), m.q);
    }
    u64 *o0 = E + (((size_t)b * 2) * ne + j) * N + x0, *o1 = o0 + (size_t)ne * N;
#pragma unroll
    for (int u = 0; u < kElems; ++u) { o0[u * blockDim.x] = e0[u]; o1[u * blockDim.x] = e1[u]; }
}
// ---- the same sum with the masks folded into the switching keys ----
// sum_dg digit_dg * (mask * key_dg) = mask * sum_dg digit_dg * key_dg modulo q, so a key multiplied by the mask once
// (k_mask_key) turns the masked pair of rotations into ONE lazy inner product with ONE reduction per output residue;
// the residues are those of k_ks_inner_pair.
// mkey[dg][p][j][i] = (mask[j][i] + mask2[j][i]) * key[dg][p][prime(j)][i];  grid = (N/(256*kElems), ne, nd*2)
__global__ void k_mask_key(u64 *__restrict__ mkey, const u64 *__restrict__ key, int key_primes, const u64 *__restrict__ mask, const u64 *__restrict__ mask2,
                           const KsPlan *__restrict__ pl, const PrimeConst *__restrict__ pc, int N) {
    const int j = blockIdx.y, dgp = blockIdx.z, ne = pl->ne;
    const int pj = pl->ext_prime[j];
    const PrimeConst m = pc[pj];
#pragma unroll
    for (int u_ = 0; u_ < kElems; ++u_) {
        const int i = (blockIdx.x * kElems + u_) * blockDim.x + threadIdx.x;
        if (i >= N) break;
        u64 w = mask[(size_t)j * N + i];
        if (mask2) w = add_mod(w, mask2[(size_t)j * N + i], m.q);
        mkey[((size_t)dgp * ne + j) * N + i] = mul_mod_any(w, key[((size_t)dgp * key_primes + pj) * N + i], m);
    }
}
// pm[j][i] = P * (mask[j][i] + mask2[j][i]) mod q_j for the Q limbs;  grid = (N/(256*kElems), n)
__global__ void k_mask_p(u64 *__restrict__ pm, const u64 *__restrict__ mask, const u64 *__restrict__ mask2, const DivPlan *__restrict__ dv, const PrimeConst *__restrict__ pc, int N) {
    const int j = blockIdx.y;
    const PrimeConst m = pc[j];
#pragma unroll
    for (int u_ = 0; u_ < kElems; ++u_) {
        const int i = (blockIdx.x * kElems + u_) * blockDim.x + threadIdx.x;
        if (i >= N) break;
        u64 w = mask[(size_t)j * N + i];
        if (mask2) w = add_mod(w, mask2[(size_t)j * N + i], m.q);
        pm[(size_t)j * N + i] = mul_mod_any(w, dv->p_mod[j], m);
    }
}
struct MaskedRot {
    const u64 *mkey[2];   // [nd][2][ne][N]
    const u64 *pm[2];     // [n][N]
    u32 g[2];
    int count;            // 1 or 2 rotations
};
constexpr int kMaxRotGroups = 16;
struct MaskedRotList { MaskedRot r[kMaxRotGroups]; }; // one entry per wrapped copy made by the same launch
// E[b][p][j][i] = sum_r sum_dg digit_dg[j][perm_r(i)] * mkey_r[dg][p][j][i]  +  (p == 0, j < n) sum_r c0[b][j][perm_r(i)] * pm_r[j][i]
// grid = (N/(256*EL), groups * batch, ne); EL coefficients per thread.  Output member g * batch + b is wrapped copy
// number g (its own pair of masked keys) of input member b: several iterations of a shift loop in one launch.
template <int EL>
__global__ void __launch_bounds__(256, EL == 2 ? 3 : 2) k_ks_inner_mk(u64 *__restrict__ E, const u64 *__restrict__ c0, const u64 *__restrict__ a_ntt, size_t a_outer, const u64 *__restrict__ dt, MaskedRotList mrl,
                              int batch, const KsPlan *__restrict__ pl, const PrimeConst *__restrict__ pc, int logn, int N) {
    const int j = blockIdx.z, ob = blockIdx.y, b = ob % batch; // limb-major block order: the key limbs stay in L2 across the members
    const MaskedRot &mr = mrl.r[ob / batch];
    const int pj = pl->ext_prime[j], nd = pl->nd, ne = pl->ne, n = pl->n;
    const PrimeConst m = pc[pj];
    const u32 x0 = blockIdx.x * (blockDim.x * EL) + threadIdx.x;
    const u64 *abase = a_ntt + (size_t)b * a_outer + (size_t)j * N;
    const u64 *cbase = c0 + (size_t)b * a_outer + (size_t)j * N;
    const u64 *dbase = dt + (size_t)b * pl->dt_count * N;
    const size_t kpoly = (size_t)ne * N;
    u64 r0[EL], r1[EL];
    if (m.fp) { // products on the FP64 pipe, signed double sums
        const double qd = (double)m.q;
        double d0[EL], d1[EL];
#pragma unroll
        for (int u = 0; u < EL; ++u) { d0[u] = 0.0; d1[u] = 0.0; }
        for (int r = 0; r < mr.count; ++r) {
            u32 src[EL];
#pragma unroll
            for (int u = 0; u < EL; ++u) src[u] = ntt_perm(x0 + u * blockDim.x, mr.g[r], logn);
            const u64 *kbase = mr.mkey[r] + (size_t)j * N + x0;
            for (int dg = 0; dg < nd; ++dg) {
                const int en = pl->dt_entry[dg][j];
                const u64 *sp = en < 0 ? abase : dbase + (size_t)en * N;
                const u64 *k0 = kbase + (size_t)dg * 2 * kpoly;
#pragma unroll
                for (int u = 0; u < EL; ++u) {
                    const double vd = u52_to_double(sp[src[u]]);
                    d0[u] = __dadd_rn(d0[u], mul_fp64_lazy(vd, u52_to_double(k0[u * blockDim.x]), m.q_inv_f, qd));
                    d1[u] = __dadd_rn(d1[u], mul_fp64_lazy(vd, u52_to_double(k0[kpoly + u * blockDim.x]), m.q_inv_f, qd));
                }
            }
            if (j < n) {
                const u64 *pmb = mr.pm[r] + (size_t)j * N + x0;
#pragma unroll
                for (int u = 0; u < EL; ++u) d0[u] = __dadd_rn(d0[u], mul_fp64_lazy(u52_to_double(cbase[src[u]]), u52_to_double(pmb[u * blockDim.x]), m.q_inv_f, qd));
            }
        }
#pragma unroll
        for (int u = 0; u < EL; ++u) { r0[u] = canon_fp64(d0[u], m.q_inv_f, qd); r1[u] = canon_fp64(d1[u], m.q_inv_f, qd); }
    } else {
        Acc128 s0[EL], s1[EL];
#pragma unroll
        for (int u = 0; u < EL; ++u) { s0[u].zero(); s1[u].zero(); }
        for (int r = 0; r < mr.count; ++r) {
            u32 src[EL];
#pragma unroll
            for (int u = 0; u < EL; ++u) src[u] = ntt_perm(x0 + u * blockDim.x, mr.g[r], logn);
            const u64 *kbase = mr.mkey[r] + (size_t)j * N + x0;
            for (int dg = 0; dg < nd; ++dg) {
                const int en = pl->dt_entry[dg][j];
                const u64 *sp = en < 0 ? abase : dbase + (size_t)en * N;
                const u64 *k0 = kbase + (size_t)dg * 2 * kpoly;
#pragma unroll
                for (int u = 0; u < EL; ++u) {
                    const u64 v = sp[src[u]];
                    s0[u].mad(v, k0[u * blockDim.x]);
                    s1[u].mad(v, k0[kpoly + u * blockDim.x]);
                }
            }
            if (j < n) {
                const u64 *pmb = mr.pm[r] + (size_t)j * N + x0;
#pragma unroll
                for (int u = 0; u < EL; ++u) s0[u].mad(cbase[src[u]], pmb[u * blockDim.x]);
            }
        }
#pragma unroll
        for (int u = 0; u < EL; ++u) { r0[u] = barrett128(s0[u].hi, s0[u].lo, m); r1[u] = barrett128(s1[u].hi, s1[u].lo, m); }
    }
    u64 *o0 = E + (((size_t)ob * 2) * ne + j) * N + x0, *o1 = o0 + (size_t)ne * N;
#pragma unroll
    for (int u = 0; u < EL; ++u) { o0[u * blockDim.x] = r0[u]; o1[u * blockDim.x] = r1[u]; }
}
// The same sums fed by bulk copies.  The automorphism maps every aligned block of 2^k outputs onto one aligned block
// of 2^k inputs, so a CTA that owns T consecutive coefficients of limb j needs, per (member, rotation, digit), exactly
// one contiguous chunk of T words -- and one chunk per key word.  One warp issues all those copies at once (tens of KB
// per CTA in flight from its first instruction on, which 8-byte register loads cannot keep up), every thread then
// waits on the mbarrier and works from shared memory: the permutation becomes an index into the staged chunk, key
// words are read once and meet M members.  Other resident CTAs of the SM compute while this one's copies land.
// Dynamic shared memory: (count*nd*2 + count + M*count*(nd+1)) * T words, count = most rotations of any group.
// grid = (N / T, groups * ceil(batch / M), ne), T = 256 * EL
template <int M, int EL>
__global__ void __launch_bounds__(256) k_ks_inner_mkb(u64 *__restrict__ E, const u64 *__restrict__ c0, const u64 *__restrict__ a_ntt, size_t a_outer, const u64 *__restrict__ dt,
                                                      const __grid_constant__ MaskedRotList mrl, int batch, int maxcount, const KsPlan *__restrict__ pl, const PrimeConst *__restrict__ pc, int logn,
                                                      int N, int *__restrict__ err) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ __align__(8) u64 bar;
    constexpr int T = 256 * EL;
    const int chunks = (batch + M - 1) / M;
    const int j = blockIdx.z, grp = blockIdx.y / chunks, b0 = (blockIdx.y % chunks) * M;
    const int nm = min(M, batch - b0);
    const MaskedRot &mr = mrl.r[grp];
    const int pj = pl->ext_prime[j], nd = pl->nd, ne = pl->ne, n = pl->n, count = mr.count;
    const bool has_c0 = j < n;
    const int nsrc = nd + 1; // chunks per (member, rotation): the digits, then c0 (left empty on the limbs of P)
    u64 *keyb = reinterpret_cast<u64 *>(smem_raw), *pmb = keyb + (size_t)maxcount * nd * 2 * T, *srcb = pmb + (size_t)maxcount * T;
    const u32 tile0 = blockIdx.x * T;
    const int tid = threadIdx.x;
    if (tid == 0) { mbar_init(&bar, 1); mbar_fence_init(); }
    __syncthreads();
    if (tid < 32) {
        const int nkey = count * nd * 2, npm = has_c0 ? count : 0, per_member = count * (nd + (has_c0 ? 1 : 0));
        const int total = nkey + npm + nm * per_member;
        if (tid == 0) mbar_arrive_expect_tx(&bar, (u32)total * T * 8);
        __syncwarp();
        for (int ci = tid; ci < total; ci += 32) {
            const u64 *src;
            u64 *dst;
            if (ci < nkey) {
                const int r = ci / (nd * 2), rem = ci % (nd * 2); // rem = digit * 2 + poly
                src = mr.mkey[r] + ((size_t)rem * ne + j) * N + tile0;
                dst = keyb + (size_t)ci * T;
            } else if (ci < nkey + npm) {
                const int r = ci - nkey;
                src = mr.pm[r] + (size_t)j * N + tile0;
                dst = pmb + (size_t)r * T;
            } else {
                const int k = ci - nkey - npm, u = k / per_member, rem = k % per_member, r = rem % count, dg = rem / count;
                const u32 st0 = ntt_perm(tile0, mr.g[r], logn) & ~(u32)(T - 1);
                if (dg < nd) {
                    const int en = pl->dt_entry[dg][j];
                    src = en < 0 ? a_ntt + (size_t)(b0 + u) * a_outer + (size_t)j * N : dt + ((size_t)(b0 + u) * pl->dt_count + en) * N;
                } else src = c0 + (size_t)(b0 + u) * a_outer + (size_t)j * N;
                src += st0;
                dst = srcb + ((size_t)(u * count + r) * nsrc + dg) * T;
            }
            bulk_load(dst, src, T * 8, &bar);
        }
    }
    mbar_wait_bounded(&bar, 0, err);
    const PrimeConst m = pc[pj];
    u64 r0[M][EL], r1[M][EL];
    if (m.fp) { // products on the FP64 pipe, signed double sums of at most 2 * (nd + 1) terms
        const double qd = (double)m.q;
        double d0[M][EL], d1[M][EL];
#pragma unroll
        for (int u = 0; u < M; ++u)
#pragma unroll
            for (int e = 0; e < EL; ++e) { d0[u][e] = 0.0; d1[u][e] = 0.0; }
        for (int r = 0; r < count; ++r) {
            u32 li[EL];
#pragma unroll
            for (int e = 0; e < EL; ++e) li[e] = ntt_perm(tile0 + e * 256 + tid, mr.g[r], logn) & (u32)(T - 1);
            for (int dg = 0; dg < nd; ++dg) {
                const u64 *kp = keyb + (size_t)((r * nd + dg) * 2) * T + tid;
                const u64 *sp = srcb + (size_t)(r * nsrc + dg) * T;
#pragma unroll
                for (int e = 0; e < EL; ++e) {
                    const double kad = u52_to_double(kp[e * 256]), kbd = u52_to_double(kp[T + e * 256]);
#pragma unroll
                    for (int u = 0; u < M; ++u)
                        if (u < nm) {
                            const double vd = u52_to_double(sp[(size_t)u * count * nsrc * T + li[e]]);
                            d0[u][e] = __dadd_rn(d0[u][e], mul_fp64_lazy(vd, kad, m.q_inv_f, qd));
                            d1[u][e] = __dadd_rn(d1[u][e], mul_fp64_lazy(vd, kbd, m.q_inv_f, qd));
                        }
                }
            }
            if (has_c0) {
                const u64 *sp = srcb + (size_t)(r * nsrc + nd) * T;
#pragma unroll
                for (int e = 0; e < EL; ++e) {
                    const double pmd = u52_to_double(pmb[(size_t)r * T + e * 256 + tid]);
#pragma unroll
                    for (int u = 0; u < M; ++u)
                        if (u < nm) d0[u][e] = __dadd_rn(d0[u][e], mul_fp64_lazy(u52_to_double(sp[(size_t)u * count * nsrc * T + li[e]]), pmd, m.q_inv_f, qd));
                }
            }
        }
#pragma unroll
        for (int u = 0; u < M; ++u)
#pragma unroll
            for (int e = 0; e < EL; ++e) { r0[u][e] = canon_fp64(d0[u][e], m.q_inv_f, qd); r1[u][e] = canon_fp64(d1[u][e], m.q_inv_f, qd); }
    } else {
        Acc128 s0[M][EL], s1[M][EL];
#pragma unroll
        for (int u = 0; u < M; ++u)
#pragma unroll
            for (int e = 0; e < EL; ++e) { s0[u][e].zero(); s1[u][e].zero(); }
        for (int r = 0; r < count; ++r) {
            u32 li[EL];
#pragma unroll
            for (int e = 0; e < EL; ++e) li[e] = ntt_perm(tile0 + e * 256 + tid, mr.g[r], logn) & (u32)(T - 1);
            for (int dg = 0; dg < nd; ++dg) {
                const u64 *kp = keyb + (size_t)((r * nd + dg) * 2) * T + tid;
                const u64 *sp = srcb + (size_t)(r * nsrc + dg) * T;
#pragma unroll
                for (int e = 0; e < EL; ++e) {
                    const u64 ka = kp[e * 256], kb = kp[T + e * 256];
#pragma unroll
                    for (int u = 0; u < M; ++u)
                        if (u < nm) {
                            const u64 v = sp[(size_t)u * count * nsrc * T + li[e]];
                            s0[u][e].mad(v, ka);
                            s1[u][e].mad(v, kb);
                        }
                }
            }
            if (has_c0) {
                const u64 *sp = srcb + (size_t)(r * nsrc + nd) * T;
#pragma unroll
                for (int e = 0; e < EL; ++e) {
                    const u64 pmv = pmb[(size_t)r * T + e * 256 + tid];
#pragma unroll
                    for (int u = 0; u < M; ++u)
                        if (u < nm) s0[u][e].mad(sp[(size_t)u * count * nsrc * T + li[e]], pmv);
                }
            }
        }
#pragma unroll
        for (int u = 0; u < M; ++u)
#pragma unroll
            for (int e = 0; e < EL; ++e) { r0[u][e] = barrett128(s0[u][e].hi, s0[u][e].lo, m); r1[u][e] = barrett128(s1[u][e].hi, s1[u][e].lo, m); }
    }
    const size_t kpoly = (size_t)ne * N;
    u64 *o0 = E + (((size_t)(grp * batch + b0) * 2) * ne + j) * N + tile0 + tid;
#pragma unroll
    for (int u = 0; u < M; ++u)
        if (u < nm) {
#pragma unroll
            for (int e = 0; e < EL; ++e) { o0[(size_t)u * 2 * kpoly + e * 256] = r0[u][e]; o0[(size_t)u * 2 * kpoly + kpoly + e * 256] = r1[u][e]; }
        }
}
// Base conversion of the division: src [bp][ns][N] (limbs q_level, P; coefficient form) -> t [bp][level][N]
// grid = (N/256, 1, nbp)
// prescaled: the inverse transform that produced src already multiplied limb k by hat_inv[k]
template <int NS>
__device__ __forceinline__ void div_conv_body(u64 *__restrict__ t, const u64 *__restrict__ src, const DivPlan *__restrict__ dv, const PrimeConst *__restrict__ pc, int N, int i, int bp,
                                              int prescaled) {
    const int nl = dv->level;
    u64 y[NS];
#pragma unroll
    for (int k = 0; k < NS; ++k) {
        const u64 v = src[((size_t)bp * NS + k) * N + i];
        y[k] = prescaled ? v : mul_shoup(v, dv->hat_inv[k], dv->hat_inv_sh[k], pc[dv->src_prime[k]].q);
    }
    u64 *o = t + (size_t)bp * nl * N + i;
    // targets below 2^44: y = y1 * 2^30 + y0 with both pieces as doubles, products on the FP64 pipe against the constants
    // (D / d_s) and (D / d_s) * 2^30 mod q: sixteen exact products of at most 0.51 q each, one canonicalisation
    double y0[NS], y1[NS];
#pragma unroll
    for (int k = 0; k < NS; ++k) {
        y0[k] = __hiloint2double(0x43300000, (int)((u32)y[k] & 0x3FFFFFFFu)) - kTwo52;
        y1[k] = __hiloint2double(0x43300000, (int)(u32)(y[k] >> 30)) - kTwo52;
    }
    for (int l = 0; l < nl; ++l) {
        if (pc[l].fp) {
            const double qinv = pc[l].q_inv_f, qd = (double)pc[l].q;
            double acc = 0.0;
#pragma unroll
            for (int k = 0; k < NS; ++k) {
                acc = __dadd_rn(acc, mul_fp64_lazy(y0[k], __longlong_as_double((long long)dv->hat_mod_d0[k][l]), qinv, qd));
                acc = __dadd_rn(acc, mul_fp64_lazy(y1[k], __longlong_as_double((long long)dv->hat_mod_d1[k][l]), qinv, qd));
            }
            *o = canon_fp64(acc, qinv, qd);
        } else {
            PieceAcc s; s.zero();
#pragma unroll
            for (int k = 0; k < NS; ++k) s.mac(y[k], dv->hat_mod[k][l]);
            PrimeConst mm; mm.q = pc[l].q; mm.mu_hi = pc[l].mu_hi; mm.mu_lo = pc[l].mu_lo;
            *o = s.finish(mm);
        }
        o += N;
    }
}
__global__ void k_div_conv(u64 *__restrict__ t, const u64 *__restrict__ src, const DivPlan *__restrict__ dv, const PrimeConst *__restrict__ pc, int N, int prescaled) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= N) return;
    const int bp = blockIdx.z;
    switch (dv->ns) {
    case 2: div_conv_body<2>(t, src, dv, pc, N, i, bp, prescaled); break;
    case 3: div_conv_body<3>(t, src, dv, pc, N, i, bp, prescaled); break;
    case 4: div_conv_body<4>(t, src, dv, pc, N, i, bp, prescaled); break;
    case 5: div_conv_body<5>(t, src, dv, pc, N, i, bp, prescaled); break;
    case 6: div_conv_body<6>(t, src, dv, pc, N, i, bp, prescaled); break;
    case 7: div_conv_body<7>(t, src, dv, pc, N, i, bp, prescaled); break;
    default: div_conv_body<8>(t, src, dv, pc, N, i, bp, prescaled); break;
    }
}
// out[bp][l][i] = (E[bp][l][i] - t[bp][l][i]) * D^-1 for l < level.  grid = (N/(256*kElems), level, batch*2)
__global__ void k_div_fin(u64 *__restrict__ out, const u64 *__restrict__ E, const u64 *__restrict__ t, int ne, const DivPlan *__restrict__ dv,
                          const PrimeConst *__restrict__ pc, int N) {
    const int l = blockIdx.y, bp = blockIdx.z, nl = dv->level;
    const PrimeConst m = pc[l];
    const u64 dinv = dv->d_inv[l];
#pragma unroll
    for (int u_ = 0; u_ < kElems; ++u_) {
        const int i = (blockIdx.x * kElems + u_) * blockDim.x + threadIdx.x;
        if (i >= N) break;
        const u64 v = sub_mod(E[((size_t)bp * ne + l) * N + i], t[((size_t)bp * nl + l) * N + i], m.q);
        out[((size_t)bp * nl + l) * N + i] = mul_mod_any(v, dinv, m);
    }
}

// ---------------- ChaCha20 ----------------
__device__ __forceinline__ u32 rotl32(u32 v, int c) { return __funnelshift_l(v, v, c); }
#define HB_QR(a, b, c, d)                                   \
    a += b; d ^= a; d = rotl32(d, 16); c += d; b ^= c; b = rotl32(b, 12); \
    a += b; d ^= a; d = rotl32(d, 8);  c += d; b ^= c; b = rotl32(b, 7);
struct ChaChaKey { u32 k[8]; };
__device__ __forceinline__ void chacha_block(const ChaChaKey &key, u32 domain, u64 id, u32 counter, u32 (&o)[16]) {
    u32 in[16] = {0x61707865u, 0x3320646eu, 0x79622d32u, 0x6b206574u, key.k[0], key.k[1], key.k[2], key.k[3], key.k[4], key.k[5], key.k[6], key.k[7],
                  counter, domain, (u32)id, (u32)(id >> 32)};
    u32 x0 = in[0], x1 = in[1], x2 = in[2], x3 = in[3], x4 = in[4], x5 = in[5], x6 = in[6], x7 = in[7];
    u32 x8 = in[8], x9 = in[9], x10 = in[10], x11 = in[11], x12 = in[12], x13 = in[13], x14 = in[14], x15 = in[15];
#pragma unroll
    for (int r = 0; r < 10; ++r) {
        HB_QR(x0, x4, x8, x12) HB_QR(x1, x5, x9, x13) HB_QR(x2, x6, x10, x14) HB_QR(x3, x7, x11, x15)
        HB_QR(x0, x5, x10, x15) HB_QR(x1, x6, x11, x12) HB_QR(x2, x7, x8, x13) HB_QR(x3, x4, x9, x14)
    }
    o[0] = x0 + in[0]; o[1] = x1 + in[1]; o[2] = x2 + in[2]; o[3] = x3 + in[3]; o[4] = x4 + in[4]; o[5] = x5 + in[5]; o[6] = x6 + in[6]; o[7] = x7 + in[7];
    o[8] = x8 + in[8]; o[9] = x9 + in[9]; o[10] = x10 + in[10]; o[11] = x11 + in[11]; o[12] = x12 + in[12]; o[13] = x13 + in[13]; o[14] = x14 + in[14]; o[15] = x15 + in[15];
}
// uniform residues: limb instance li (prime pi = map.prime[li]) coefficient c = (128-bit word (pi*N + c) of the stream) mod q.
// One thread produces the four coefficients of one ChaCha block.  grid = (N/4/256, count)
__global__ void k_uniform(u64 *__restrict__ out, LimbMap map, const PrimeConst *__restrict__ pc, int N, ChaChaKey key, u32 domain, u64 id) {
    const int li = blockIdx.y;
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t * 4 >= N) return;
    const int pi = map.prime[li % map.n];
    const PrimeConst m = pc[pi];
    u32 o[16];
    chacha_block(key, domain, id, (u32)(((u64)pi * N + (u64)t * 4) >> 2), o);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        u64 lo = (u64)o[4 * k] | ((u64)o[4 * k + 1] << 32), hi = (u64)o[4 * k + 2] | ((u64)o[4 * k + 3] << 32);
        out[(size_t)li * N + t * 4 + k] = barrett128(hi, lo, m);
    }
}

// ---------------- encrypt / decrypt / key generation ----------------
// b = e - a*s + msg   (all NTT form).  grid.y = n limbs
__global__ void k_encrypt(u64 *__restrict__ b, const u64 *__restrict__ a, const u64 *__restrict__ e, const u64 *__restrict__ s, const u64 *__restrict__ msg, LimbMap map,
                          const PrimeConst *__restrict__ pc, int N) {
    const int li = blockIdx.y;
#pragma unroll
    for (int u_ = 0; u_ < kElems; ++u_) {
        const int i = (blockIdx.x * kElems + u_) * blockDim.x + threadIdx.x;
        if (i >= N) break;
        const PrimeConst m = pc[map.prime[li % map.n]];
        const size_t off = (size_t)li * N + i;
        const size_t so = (size_t)map.prime[li % map.n] * N + i;
        u64 v = sub_mod(e[off], mul_mod(a[off], s[so], m), m.q);
        b[off] = add_mod(v, msg[off], m.q);
    }
}
// out[l] = b + a*s (+ d2*s^2) for limbs l < nl of entry `index`
__global__ void k_decrypt(u64 *__restrict__ out, const u64 *__restrict__ ct, int n, int np, const u64 *__restrict__ s, const PrimeConst *__restrict__ pc, int N) {
    const int l = blockIdx.y;
#pragma unroll
    for (int u_ = 0; u_ < kElems; ++u_) {
        const int i = (blockIdx.x * kElems + u_) * blockDim.x + threadIdx.x;
        if (i >= N) break;
        const PrimeConst m = pc[l];
        const u64 sv = s[(size_t)l * N + i];
        u64 v = add_mod(ct[(size_t)l * N + i], mul_mod(ct[((size_t)n + l) * N + i], sv, m), m.q);
        if (np == 3) v = add_mod(v, mul_mod(ct[((size_t)2 * n + l) * N + i], mul_mod(sv, sv, m), m), m.q);
        out[(size_t)l * N + i] = v;
    }
}
// switching-key body: b = e - a*s + [prime in digit] * (P mod q) * s',  s' = s^2 (g == 0) or s o perm_g.
// grid.y = nprimes; one digit per launch.
__global__ void k_keygen(u64 *__restrict__ b, const u64 *__restrict__ a, const u64 *__restrict__ e, const u64 *__restrict__ s, const PrimeConst *__restrict__ pc, int N,
                         int logn, u32 g, int dig_lo, int dig_hi, Scalars pmod) {
    const int pi = blockIdx.y;
#pragma unroll
    for (int u_ = 0; u_ < kElems; ++u_) {
        const int i = (blockIdx.x * kElems + u_) * blockDim.x + threadIdx.x;
        if (i >= N) break;
        const PrimeConst m = pc[pi];
        const size_t off = (size_t)pi * N + i;
        u64 v = sub_mod(e[off], mul_mod(a[off], s[off], m), m.q);
        if (pi >= dig_lo && pi < dig_hi) {
            u64 sp;
            if (g == 0) sp = mul_mod(s[off], s[off], m);
            else sp = s[(size_t)pi * N + ntt_perm((u32)i, g, logn)];
            v = add_mod(v, mul_mod(sp, pmod.v[pi], m), m.q);
        }
        b[off] = v;
    }
}

// ---------------- fused plaintext-matmul accumulate ----------------
// out[p][l][i] = sum_{b < bcount} sum_{k < kcount} pre[k * btotal + b0 + b][p][l][i] * pt_b[l][perm_{g_k}(i)]
// (scale Delta^2, no rescale).  Shifted copies are stored k-major; the sum over b adds the partial products
// of several K-groups in the same pass.  grid = (N/256, 2*n).  The 128-bit accumulator is folded every 64 terms.
struct PtList { const u64 *p[16]; };
__global__ void k_matmul_acc(u64 *__restrict__ out, const u64 *__restrict__ pre, int kcount, int btotal, int b0, int bcount, PtList pts, const u32 *__restrict__ gal,
                             int n, LimbMap map, const PrimeConst *__restrict__ pc, int logn, int N) {
    const int pl = blockIdx.y, l = pl % n;
    const PrimeConst m = pc[map.prime[l]];
    const size_t estride = (size_t)2 * n * N;
    const u32 x0 = blockIdx.x * (blockDim.x * kElems) + threadIdx.x;
    const u64 *pbase = pre + (size_t)pl * N + x0;
    u64 total[kElems];
#pragma unroll
    for (int u = 0; u < kElems; ++u) total[u] = 0;
    // the four coefficients of a thread sit in the inner loop: their loads (and those of the next K-group) overlap
    if (m.fp) { // lazy terms below 1.6q: the running sum is folded before it can reach 2^52 (reduce_fp's input range)
        u64 acc[kElems];
#pragma unroll
        for (int u = 0; u < kElems; ++u) acc[u] = 0;
        int terms = 0;
        const int fold_at = (int)m.lazy_terms - 16; // a round of the inner loop adds at most 16 terms (bcount <= 16)
        for (int k = 0; k < kcount; ++k) {
            const u32 g = __ldg(gal + k);
            u32 src[kElems];
#pragma unroll
            for (int u = 0; u < kElems; ++u) src[u] = g == 1 ? x0 + u * blockDim.x : ntt_perm(x0 + u * blockDim.x, g, logn);
#pragma unroll 2
            for (int b = 0; b < bcount; ++b) {
                const u64 *a = pbase + ((size_t)k * btotal + b0 + b) * estride, *w = pts.p[b] + (size_t)l * N;
#pragma unroll
                for (int u = 0; u < kElems; ++u) acc[u] += mul_small_lazy(a[u * blockDim.x], w[src[u]], m.q_inv_f, m.q);
            }
            terms += bcount;
            if (terms > fold_at) {
#pragma unroll
                for (int u = 0; u < kElems; ++u) { total[u] = add_mod(total[u], reduce_fp(acc[u], m.q_inv_f, m.q), m.q); acc[u] = 0; }
                terms = 0;
            }
        }
#pragma unroll
        for (int u = 0; u < kElems; ++u) total[u] = add_mod(total[u], reduce_fp(acc[u], m.q_inv_f, m.q), m.q);
    } else {
        Acc128 s[kElems];
#pragma unroll
        for (int u = 0; u < kElems; ++u) s[u].zero();
        int terms = 0;
        for (int k = 0; k < kcount; ++k) {
            const u32 g = __ldg(gal + k);
            u32 src[kElems];
#pragma unroll
            for (int u = 0; u < kElems; ++u) src[u] = g == 1 ? x0 + u * blockDim.x : ntt_perm(x0 + u * blockDim.x, g, logn);
#pragma unroll 2
            for (int b = 0; b < bcount; ++b) {
                const u64 *a = pbase + ((size_t)k * btotal + b0 + b) * estride, *w = pts.p[b] + (size_t)l * N;
#pragma unroll
                for (int u = 0; u < kElems; ++u) s[u].mad(a[u * blockDim.x], w[src[u]]);
            }
            terms += bcount;
            if (terms >= 48) { // products below 2^120: the 128-bit accumulator holds 256 of them
#pragma unroll
                for (int u = 0; u < kElems; ++u) { total[u] = add_mod(total[u], barrett128(s[u].hi, s[u].lo, m), m.q); s[u].zero(); }
                terms = 0;
            }
        }
#pragma unroll
        for (int u = 0; u < kElems; ++u) total[u] = add_mod(total[u], barrett128(s[u].hi, s[u].lo, m), m.q);
    }
    u64 *op = out + (size_t)pl * N + x0;
#pragma unroll
    for (int u = 0; u < kElems; ++u) op[u * blockDim.x] = total[u];
}

// The same for T output tiles that share the shifted copies: a copy word is read once and meets the weights of T tiles
// (all output tiles of a sublayer multiply the same copies of x), so the copies -- the bulk of the traffic -- cross HBM
// once per T tiles.  Two coefficients per thread.  Primes below 2^44: products on the FP64 pipe, signed double sums folded
// every 512 terms (512 * 0.51 q stays far below 2^53).  grid = (N/512, 2*n)
template <int T> struct TilePts { const u64 *p[T][16]; u64 *out[T]; };
template <int T>
__global__ void __launch_bounds__(256) k_matmul_acc_tiles(const __grid_constant__ TilePts<T> tp, const u64 *__restrict__ pre, int kcount, int btotal, int b0, int bcount,
                                                          const u32 *__restrict__ gal, int n, const __grid_constant__ LimbMap map, const PrimeConst *__restrict__ pc, int logn, int N) {
    constexpr int E = 2;
    const int pl = blockIdx.y, l = pl % n;
    const PrimeConst m = pc[map.prime[l]];
    const size_t estride = (size_t)2 * n * N;
    const u32 x0 = blockIdx.x * (blockDim.x * E) + threadIdx.x;
    const u64 *pbase = pre + (size_t)pl * N + x0;
    u64 total[T][E];
#pragma unroll
    for (int t = 0; t < T; ++t)
#pragma unroll
        for (int u = 0; u < E; ++u) total[t][u] = 0;
    if (m.fp) {
        const double qd = (double)m.q;
        double acc[T][E];
#pragma unroll
        for (int t = 0; t < T; ++t)
#pragma unroll
            for (int u = 0; u < E; ++u) acc[t][u] = 0.0;
        int terms = 0;
        for (int k = 0; k < kcount; ++k) {
            const u32 g = __ldg(gal + k);
            u32 src[E];
#pragma unroll
            for (int u = 0; u < E; ++u) src[u] = g == 1 ? x0 + u * blockDim.x : ntt_perm(x0 + u * blockDim.x, g, logn);
            for (int b = 0; b < bcount; ++b) {
                const u64 *a = pbase + ((size_t)k * btotal + b0 + b) * estride;
                double ad[E];
#pragma unroll
                for (int u = 0; u < E; ++u) ad[u] = u52_to_double(a[u * blockDim.x]);
#pragma unroll
                for (int t = 0; t < T; ++t) {
                    const u64 *w = tp.p[t][b] + (size_t)l * N;
#pragma unroll
                    for (int u = 0; u < E; ++u) acc[t][u] = __dadd_rn(acc[t][u], mul_fp64_lazy(ad[u], u52_to_double(w[src[u]]), m.q_inv_f, qd));
                }
            }
            terms += bcount;
            if (terms >= 496) {
#pragma unroll
                for (int t = 0; t < T; ++t)
#pragma unroll
                    for (int u = 0; u < E; ++u) { total[t][u] = add_mod(total[t][u], canon_fp64(acc[t][u], m.q_inv_f, qd), m.q); acc[t][u] = 0.0; }
                terms = 0;
            }
        }
#pragma unroll
        for (int t = 0; t < T; ++t)
#pragma unroll
            for (int u = 0; u < E; ++u) total[t][u] = add_mod(total[t][u], canon_fp64(acc[t][u], m.q_inv_f, qd), m.q);
    } else {
        Acc128 s[T][E];
#pragma unroll
        for (int t = 0; t < T; ++t)
#pragma unroll
            for (int u = 0; u < E; ++u) s[t][u].zero();
        int terms = 0;
        for (int k = 0; k < kcount; ++k) {
            const u32 g = __ldg(gal + k);
            u32 src[E];
#pragma unroll
            for (int u = 0; u < E; ++u) src[u] = g == 1 ? x0 + u * blockDim.x : ntt_perm(x0 + u * blockDim.x, g, logn);
            for (int b = 0; b < bcount; ++b) {
                const u64 *a = pbase + ((size_t)k * btotal + b0 + b) * estride;
                u64 av[E];
#pragma unroll
                for (int u = 0; u < E; ++u) av[u] = a[u * blockDim.x];
#pragma unroll
                for (int t = 0; t < T; ++t) {
                    const u64 *w = tp.p[t][b] + (size_t)l * N;
#pragma unroll
                    for (int u = 0; u < E; ++u) s[t][u].mad(av[u], w[src[u]]);
                }
            }
            terms += bcount;
            if (terms >= 48) { // products below 2^120: the 128-bit accumulator holds 256 of them
#pragma unroll
                for (int t = 0; t < T; ++t)
#pragma unroll
                    for (int u = 0; u < E; ++u) { total[t][u] = add_mod(total[t][u], barrett128(s[t][u].hi, s[t][u].lo, m), m.q); s[t][u].zero(); }
                terms = 0;
            }
        }
#pragma unroll
        for (int t = 0; t < T; ++t)
#pragma unroll
            for (int u = 0; u < E; ++u) total[t][u] = add_mod(total[t][u], barrett128(s[t][u].hi, s[t][u].lo, m), m.q);
    }
#pragma unroll
    for (int t = 0; t < T; ++t) {
        u64 *op = tp.out[t] + (size_t)pl * N + x0;
#pragma unroll
        for (int u = 0; u < E; ++u) op[u * blockDim.x] = total[t][u];
    }
}

} // namespace hb
