// A routed feed-forward (mixture of experts): the router's choice, the sort of the chosen (token, expert) pairs by
// expert, the experts' two products over those pairs, and the weighted sum per token.
//
//   scores   s_e = sigmoid(z_e), or softmax(z)_e over all router outputs, from the router's logits z (fp32); the choice is
//            made on c_e = s_e + correction_e
//   groups   the experts form n_groups equal groups of neighbours; a group's score is the sum of its two largest
//            c_e, or its largest; only experts of the `keep` best groups can be chosen (the others count as -inf)
//   choice   the `top` largest c_e (the lower index on ties)
//   weights  w = s_chosen / (sum of the chosen s + 1e-20) * scale, or s_chosen * scale   (s without the correction)
//   identity the router's last outputs may be experts without tensors whose output is their input: they take part in
//            scores, groups and choice like the others, are left out of the sort, and enter the weighted sum as w * h
//   expert   y = W_down (silu(W_gate h) * (W_up h)), no biases
//   output   out[t] = sum_k w[t, k] y_(e[t, k])(h[t])  (+ gate[t] * shared[t] for an expert every token uses)
//
// Everything a later kernel needs of the choice stays on the device (nothing is read on the host, so the step can be
// captured in a graph): the pairs ("entries", entry = token * top + k) are sorted into tiles of BM rows that belong to
// one expert each (`moe_align`: sorted[tile * BM + r] = entry or -1, tile_expert[tile] = expert or -1), and the
// products run over at most (entries + E * (BM - 1)) / BM tiles, a bound the host knows from the sizes alone.
// A row of a product is the same sum in the same order wherever the row lands, so the result does not depend on what
// else is in the batch.  All sums are fp32; the CUDA-core product serves the float32 run and shapes the tensor-core
// product refuses.
#include "common.cuh"

namespace {

constexpr int ROUTE_WARPS = 4;

// ------------------------------------------------------------------- the choice
// One warp per token.  logits [T, ld] fp32: columns [0, E) the router's, column `gate_col` (if gate != null) the
// logit of a shared expert's gate.  ids [T, top] int32, weights [T, top] fp32, gate [T] fp32 = sigmoid(that logit).
__global__ void __launch_bounds__(ROUTE_WARPS * 32)
route_topk_kernel(const float* __restrict__ logits, int ld, const float* __restrict__ correction, int E, int top,
                  int n_groups, int keep, float scale, int* __restrict__ ids, float* __restrict__ weights,
                  float* __restrict__ gate, int gate_col, int T, int softmax_scores, int group_by_max, int normalize) {
    extern __shared__ float route_sm[];             // per warp: s[E], c[E], group score[n_groups], group kept[n_groups]
    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * ROUTE_WARPS + warp;
    if (t >= T) return;                             // warp-level exit; no block barrier below
    float* s = route_sm + (size_t)warp * (2 * E + 2 * n_groups);
    float* c = s + E;
    float* gs = c + E;
    float* kept = gs + n_groups;
    const float* z = logits + (size_t)t * ld;
    float zmax = 0.f, zden = 1.f;
    if (softmax_scores) {
        // softmax over all E outputs: the maximum, then the sum of the exponentials, each in an order E alone fixes
        zmax = -INFINITY;
        for (int e = lane; e < E; e += 32) zmax = fmaxf(zmax, z[e]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) zmax = fmaxf(zmax, __shfl_xor_sync(0xffffffffu, zmax, o));
        float part = 0.f;
        for (int e = lane; e < E; e += 32) part += expf(z[e] - zmax);
        zden = warp_sum(part);
    }
    for (int e = lane; e < E; e += 32) {
        const float v = softmax_scores ? expf(z[e] - zmax) / zden : 1.0f / (1.0f + expf(-z[e]));
        float cv = v + (correction ? correction[e] : 0.f);
        if (!(cv == cv)) cv = -INFINITY;            // a NaN is never chosen before anything else
        s[e] = v;
        c[e] = cv;
    }
    __syncwarp();
    if (n_groups > 1 && keep < n_groups) {
        const int per = E / n_groups;
        for (int g = lane; g < n_groups; g += 32) {
            float a = -INFINITY, b = -INFINITY;     // the two largest of the group
            for (int j = 0; j < per; ++j) {
                const float v = c[g * per + j];
                if (v > a) { b = a; a = v; } else if (v > b) { b = v; }
            }
            gs[g] = per >= 2 && !group_by_max ? a + b : a;
            kept[g] = 0.f;
        }
        __syncwarp();
        for (int r = 0; r < keep; ++r) {
            float best = -INFINITY;
            int bi = 0x7fffffff;
            for (int g = lane; g < n_groups; g += 32) {
                if (kept[g] != 0.f) continue;
                float v = gs[g];
                if (!(v == v)) v = -INFINITY;
                if (v > best || (v == best && g < bi)) { best = v; bi = g; }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ob = __shfl_xor_sync(0xffffffffu, best, o);
                const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
            }
            if (lane == 0 && bi < n_groups) kept[bi] = 1.f;
            __syncwarp();
        }
        for (int e = lane; e < E; e += 32)
            if (kept[e / per] == 0.f) c[e] = -INFINITY;
        __syncwarp();
    }
    float sum = 0.f;
    for (int r = 0; r < top; ++r) {
        float best = -INFINITY;
        int bi = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float v = c[e];
            if (!(v == v)) continue;                // taken already
            if (v > best || (v == best && e < bi)) { best = v; bi = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
        }
        if (bi >= E) bi = 0;                        // more choices than experts: refused on the host
        const float sv = s[bi];
        sum += sv;
        if (lane == 0) {
            ids[(size_t)t * top + r] = bi;
            weights[(size_t)t * top + r] = sv;
            c[bi] = __int_as_float(0x7fc00000);     // NaN: taken
        }
        __syncwarp();
    }
    if (lane == 0) {
        const float den = sum + 1e-20f;
        for (int r = 0; r < top; ++r) {
            const float wv = weights[(size_t)t * top + r];
            weights[(size_t)t * top + r] = normalize ? wv / den * scale : wv * scale;
        }
        if (gate) gate[t] = 1.0f / (1.0f + expf(-z[gate_col]));
    }
}

// ------------------------------------------------------------------ the router's logits
// out[t, e] = sum_k h[t, k] w[e, k] in fp32 for a handful of rows of w (the experts' router rows and a gate's): four
// tokens a block with their rows of h in shared memory as fp32, a warp per row of w (blockIdx.y: which eight rows), lanes
// over k and a shuffle tree at the end, so that a logit's sum has the same order in every batch.
constexpr int RL_TOKENS = 4, RL_WARPS = 8;
__device__ __forceinline__ float4 rl_load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 rl_load4(const bf16* p) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&u.x), b = *reinterpret_cast<const __nv_bfloat162*>(&u.y);
    return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
}
template <typename Th, typename Tw>
__global__ void __launch_bounds__(RL_WARPS * 32)
router_logits_kernel(const Th* __restrict__ h, const Tw* __restrict__ w, float* __restrict__ out, int T, int E, int K) {
    extern __shared__ float rl_sm[];                // [RL_TOKENS][K]
    pdl_launch_dependents();
    pdl_wait();
    const int t0 = blockIdx.x * RL_TOKENS, nt = min(RL_TOKENS, T - t0);
#pragma unroll
    for (int tt = 0; tt < RL_TOKENS; ++tt) {
        const Th* hr = h + (size_t)(t0 + (tt < nt ? tt : 0)) * K;
        for (int k = threadIdx.x; k < K; k += RL_WARPS * 32) rl_sm[tt * K + k] = tt < nt ? to_f32<Th>(hr[k]) : 0.f;
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int e = blockIdx.y * RL_WARPS + warp; e < E; e += gridDim.y * RL_WARPS) {
        const Tw* wr = w + (size_t)e * K;
        float acc[RL_TOKENS];
#pragma unroll
        for (int tt = 0; tt < RL_TOKENS; ++tt) acc[tt] = 0.f;
        if (K % 4 == 0 && ((uintptr_t)w & 15) == 0) {
            // four consecutive k a lane and step: one 8- or 16-byte load of the weights, one 16-byte load a token
#pragma unroll 2
            for (int k = lane * 4; k < K; k += 128) {
                const float4 wv = rl_load4(wr + k);
#pragma unroll
                for (int tt = 0; tt < RL_TOKENS; ++tt) {
                    const float4 hv = *reinterpret_cast<const float4*>(rl_sm + tt * K + k);
                    acc[tt] = fmaf(hv.x, wv.x, acc[tt]);
                    acc[tt] = fmaf(hv.y, wv.y, acc[tt]);
                    acc[tt] = fmaf(hv.z, wv.z, acc[tt]);
                    acc[tt] = fmaf(hv.w, wv.w, acc[tt]);
                }
            }
        } else {
#pragma unroll 4
            for (int k = lane; k < K; k += 32) {
                const float wv = to_f32<Tw>(wr[k]);
#pragma unroll
                for (int tt = 0; tt < RL_TOKENS; ++tt) acc[tt] = fmaf(rl_sm[tt * K + k], wv, acc[tt]);
            }
        }
#pragma unroll
        for (int tt = 0; tt < RL_TOKENS; ++tt) {
            const float v = warp_sum(acc[tt]);
            if (lane == 0 && tt < nt) out[(size_t)(t0 + tt) * E + e] = v;
        }
    }
}

// ---------------------------------------------------------------------- the sort
// One block.  ids [n_entries] -> sorted [max_tiles * BM] (entry or -1), tile_expert [max_tiles] (expert or -1),
// where [n_entries] the row of `sorted` that holds the entry.  Where an entry lands inside its expert's rows depends on
// the order of the atomics; no result depends on it.  Entries whose id lies in [E, E + n_skip) (experts without
// tensors) are left out: where = -1.
constexpr int ALIGN_NT = 1024;
__global__ void __launch_bounds__(ALIGN_NT)
moe_align_kernel(const int* __restrict__ ids, int n_entries, int E, int BM, int* __restrict__ tile_expert,
                 int* __restrict__ sorted, int* __restrict__ where, int max_tiles, int n_skip) {
    extern __shared__ int align_sm[];               // cnt[E], off[E + 1], fill[E]
    pdl_launch_dependents();
    pdl_wait();
    int* cnt = align_sm;
    int* off = cnt + E;
    int* fill = off + E + 1;
    for (int e = threadIdx.x; e < E; e += ALIGN_NT) { cnt[e] = 0; fill[e] = 0; }
    __syncthreads();
    for (int i = threadIdx.x; i < n_entries; i += ALIGN_NT) {
        int e = ids[i];
        if (e >= E && e < E + n_skip) continue;
        if (e < 0 || e >= E) e = 0;
        atomicAdd(&cnt[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int o = 0;
        for (int e = 0; e < E; ++e) {
            off[e] = o;
            o += (cnt[e] + BM - 1) / BM * BM;
        }
        off[E] = o;
    }
    __syncthreads();
    for (int tile = threadIdx.x; tile < max_tiles; tile += ALIGN_NT) {
        const int row = tile * BM;
        int e = -1;
        if (row < off[E]) {
            int lo = 0, hi = E;                     // the last e with off[e] <= row
            while (hi - lo > 1) {
                const int mid = (lo + hi) >> 1;
                if (off[mid] <= row) lo = mid; else hi = mid;
            }
            e = lo;
        }
        tile_expert[tile] = e;
    }
    for (int i = threadIdx.x; i < max_tiles * BM; i += ALIGN_NT) sorted[i] = -1;
    __syncthreads();
    for (int i = threadIdx.x; i < n_entries; i += ALIGN_NT) {
        int e = ids[i];
        if (e >= E && e < E + n_skip) { where[i] = -1; continue; }
        if (e < 0 || e >= E) e = 0;
        const int p = off[e] + atomicAdd(&fill[e], 1);
        if (p < max_tiles * BM) sorted[p] = i;
        where[i] = p;
    }
}

// ------------------------------------------------------- the experts' products (CUDA cores)
// A tile of BM sorted rows times a tile of 64 columns of its expert's weights, k ascending, fp32 sums.
// MODE 0 (gate and up): row r of the tile is token sorted[...] / top of `a` [T, K]; w is [E][2 N][K], an expert's
//   N gate rows followed by its N up rows; out[tile * BM + r, n] = silu(g) * u in To.
// MODE 1 (down): row r of the tile is row tile * BM + r of `a` [max_tiles * BM, K]; w is [E][N][K];
//   out[tile * BM + r, n] = sum in fp32 (the weighted sum per token comes after).
constexpr int MG_BN = 64, MG_BK = 16;

// where gate row n and up row n of an expert lie in its [2 N, K] matrix
__device__ __forceinline__ int gate_row_of(int n, int N, int interleaved) { return interleaved ? (n >> 6) * 128 + (n & 63) : n; }
__device__ __forceinline__ int up_row_of(int n, int N, int interleaved) { return interleaved ? (n >> 6) * 128 + 64 + (n & 63) : N + n; }

template <typename Ta, typename Tw, typename To, int BM, int MODE>
__global__ void __launch_bounds__(256)
moe_gemm_kernel(const Ta* __restrict__ a, long lda, int top, const Tw* __restrict__ w, To* __restrict__ out, long ldo,
                const int* __restrict__ tile_expert, const int* __restrict__ sorted, int N, int K, int interleaved) {
    constexpr int TM = BM / 16;
    __shared__ float As[MG_BK][BM + 1];
    __shared__ float Bs[MODE == 0 ? 2 : 1][MG_BK][MG_BN + 1];
    __shared__ long a_off[BM];
    pdl_launch_dependents();
    pdl_wait();
    const int tile = blockIdx.x;
    const int e = tile_expert[tile];
    if (e < 0) return;
    const int n0 = blockIdx.y * MG_BN;
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    for (int r = tid; r < BM; r += 256) {
        const int entry = sorted[tile * BM + r];
        a_off[r] = entry < 0 ? -1 : (MODE == 0 ? (long)(entry / top) * lda : (long)(tile * BM + r) * lda);
    }
    __syncthreads();
    const Tw* wg = w + (size_t)e * (MODE == 0 ? 2 : 1) * N * K;
    float acc[MODE == 0 ? 2 : 1][TM][4];
#pragma unroll
    for (int m = 0; m < (MODE == 0 ? 2 : 1); ++m)
#pragma unroll
        for (int i = 0; i < TM; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[m][i][j] = 0.f;
    for (int k0 = 0; k0 < K; k0 += MG_BK) {
        for (int idx = tid; idx < BM * MG_BK; idx += 256) {
            const int r = idx / MG_BK, k = idx - r * MG_BK;
            const long o = a_off[r];
            As[k][r] = (o >= 0 && k0 + k < K) ? to_f32<Ta>(a[o + k0 + k]) : 0.f;
        }
        for (int idx = tid; idx < MG_BN * MG_BK; idx += 256) {
            const int n = idx / MG_BK, k = idx - n * MG_BK;
            const bool ok = n0 + n < N && k0 + k < K;
            const int row_g = MODE == 0 ? gate_row_of(n0 + n, N, interleaved) : n0 + n;
            Bs[0][k][n] = ok ? to_f32<Tw>(wg[(size_t)row_g * K + k0 + k]) : 0.f;
            if (MODE == 0) Bs[MODE == 0 ? 1 : 0][k][n] = ok ? to_f32<Tw>(wg[(size_t)up_row_of(n0 + n, N, interleaved) * K + k0 + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < MG_BK; ++k) {
            float av[TM];
#pragma unroll
            for (int i = 0; i < TM; ++i) av[i] = As[k][ty * TM + i];
#pragma unroll
            for (int m = 0; m < (MODE == 0 ? 2 : 1); ++m)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float bv = Bs[m][k][tx * 4 + j];
#pragma unroll
                    for (int i = 0; i < TM; ++i) acc[m][i][j] = fmaf(av[i], bv, acc[m][i][j]);
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int r = ty * TM + i;
        if (a_off[r] < 0) continue;
        To* o = out + (size_t)(tile * BM + r) * ldo;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            if (MODE == 0) {
                // both branches rounded to the activations' type first, as a product that stores them would
                const float g = to_f32<To>(from_f32<To>(acc[0][i][j])), u = to_f32<To>(from_f32<To>(acc[MODE == 0 ? 1 : 0][i][j]));
                o[n] = from_f32<To>(g / (1.0f + expf(-g)) * u);
            } else {
                o[n] = from_f32<To>(acc[0][i][j]);
            }
        }
    }
}

// ------------------------------------------------ the experts' products (mma.sync, few rows an expert)
// The same two products for bfloat16 where an expert has few rows (decode steps): a tile of 16 sorted rows times 64
// columns of its expert's weights on `mma.sync.m16n8k16`, fp32 sums.  The weights are what the kernel moves (every
// element is used once per tile), so they go from global memory straight into the B fragments, 16 bytes a thread and
// row (eight consecutive k: two MMA steps, with the tile's rows read from shared memory in the same order of k);
// the 16 rows sit in shared memory in pieces of 1,024 columns of K.  A row's sum has the same order wherever the row
// lands.  N a multiple of 8, K a multiple of 32.
// (measured at 8 tokens x 3 of 32 experts of 2,048 x 2,048, gate/up and down together, cold L2: one block of eight columns a
// warp and four steps of K unrolled 114 us; two blocks a warp 140 us; four 167 us; four warps a block 210 us; sixteen 118 us)
#ifndef PLM_MM_NB
#define PLM_MM_NB 1
#endif
#ifndef PLM_MM_WARPS
#define PLM_MM_WARPS 8
#endif
#ifndef PLM_MM_UNROLL
#define PLM_MM_UNROLL 4
#endif
constexpr int MM_WARPS = PLM_MM_WARPS, MM_NB = PLM_MM_NB, MM_BN = MM_WARPS * MM_NB * 8, MM_KC = 1024, MM_LD = MM_KC + 32;

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                               uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}


template <int MODE>
__global__ void __launch_bounds__(MM_WARPS * 32)
moe_gemm_mma_kernel(const bf16* __restrict__ a, long lda, int top, const bf16* __restrict__ w, void* __restrict__ out_, long ldo,
                    const int* __restrict__ tile_expert, const int* __restrict__ sorted, int N, int K, int interleaved) {
    constexpr int BM = 16, NACC = MODE == 0 ? 2 : 1;
    extern __shared__ __align__(16) uint8_t mm_raw[];
    bf16* As = reinterpret_cast<bf16*>(mm_raw);                        // [16][MM_LD]
    __shared__ long a_off[BM];
    pdl_launch_dependents();
    pdl_wait();
    const int tile = blockIdx.x;
    const int e = tile_expert[tile];
    if (e < 0) return;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, c = lane & 3;
    if (tid < BM) {
        const int entry = sorted[tile * BM + tid];
        a_off[tid] = entry < 0 ? -1 : (MODE == 0 ? (long)(entry / top) * lda : (long)(tile * BM + tid) * lda);
    }
    const bf16* we = w + (size_t)e * NACC * N * K;
    const int n_base = blockIdx.y * MM_BN + warp * MM_NB * 8;
    // the weight rows this thread reads: column n_base + 8 j + g of gate (and up)
    const bf16* wrow[NACC][MM_NB];
    bool col_ok[MM_NB];
#pragma unroll
    for (int j = 0; j < MM_NB; ++j) {
        const int n = n_base + 8 * j + g;
        col_ok[j] = n < N;
        const int nn = col_ok[j] ? n : 0;
        wrow[0][j] = we + (size_t)(MODE == 0 ? gate_row_of(nn, N, interleaved) : nn) * K + c * 8;
        if (MODE == 0) wrow[NACC - 1][j] = we + (size_t)up_row_of(nn, N, interleaved) * K + c * 8;
    }
    float acc[NACC][MM_NB][4];
#pragma unroll
    for (int m = 0; m < NACC; ++m)
#pragma unroll
        for (int j = 0; j < MM_NB; ++j) acc[m][j][0] = acc[m][j][1] = acc[m][j][2] = acc[m][j][3] = 0.f;
    __syncthreads();
    for (int kc = 0; kc < K; kc += MM_KC) {
        const int kn = min(MM_KC, K - kc);
        for (int idx = tid; idx < BM * (kn / 8); idx += MM_WARPS * 32) {
            const int r = idx / (kn / 8), k8 = idx - r * (kn / 8);
            const long o = a_off[r];
            uint4 v = make_uint4(0, 0, 0, 0);
            if (o >= 0) v = *reinterpret_cast<const uint4*>(a + o + kc + k8 * 8);
            *reinterpret_cast<uint4*>(As + r * MM_LD + k8 * 8) = v;
        }
        __syncthreads();
        if (n_base < N) {
#define PLM_PRAGMA_(x) _Pragma(#x)
#define PLM_UNROLL_(n) PLM_PRAGMA_(unroll n)
            PLM_UNROLL_(PLM_MM_UNROLL)
            for (int k0 = 0; k0 < kn; k0 += 32) {
                uint4 b[NACC][MM_NB];
#pragma unroll
                for (int m = 0; m < NACC; ++m)
#pragma unroll
                    for (int j = 0; j < MM_NB; ++j) b[m][j] = __ldg(reinterpret_cast<const uint4*>(wrow[m][j] + kc + k0));
                const uint4 lo = *reinterpret_cast<const uint4*>(As + g * MM_LD + k0 + c * 8);
                const uint4 hi = *reinterpret_cast<const uint4*>(As + (g + 8) * MM_LD + k0 + c * 8);
#pragma unroll
                for (int m = 0; m < NACC; ++m)
#pragma unroll
                    for (int j = 0; j < MM_NB; ++j) {
                        mma_bf16_16816(acc[m][j], lo.x, hi.x, lo.y, hi.y, b[m][j].x, b[m][j].y);
                        mma_bf16_16816(acc[m][j], lo.z, hi.z, lo.w, hi.w, b[m][j].z, b[m][j].w);
                    }
            }
        }
        __syncthreads();
    }
    // c0, c1: row g, columns 2 c, 2 c + 1 of the block of eight; c2, c3: row g + 8
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int r = g + 8 * half;
        if (a_off[r] < 0) continue;
#pragma unroll
        for (int j = 0; j < MM_NB; ++j) {
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int n = n_base + 8 * j + 2 * c + i;
                if (n >= N) continue;
                if (MODE == 0) {
                    const float gv = __bfloat162float(__float2bfloat16_rn(acc[0][j][2 * half + i]));
                    const float uv = __bfloat162float(__float2bfloat16_rn(acc[NACC - 1][j][2 * half + i]));
                    reinterpret_cast<bf16*>(out_)[(size_t)(tile * BM + r) * ldo + n] = __float2bfloat16_rn(gv / (1.0f + expf(-gv)) * uv);
                } else {
                    reinterpret_cast<float*>(out_)[(size_t)(tile * BM + r) * ldo + n] = acc[0][j][2 * half + i];
                }
            }
        }
    }
}

// ------------------------------------------------------------------ rows in sorted order
// dst[p, :] = src[sorted[p] / top, :] (zero where sorted[p] < 0): the tokens' rows laid out as the sorted tiles want
// them, for a product that takes whole tiles of its left operand.
__global__ void moe_gather_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, const int* __restrict__ sorted,
                                  int top, long row_bytes) {
    pdl_launch_dependents();
    pdl_wait();
    const int p = blockIdx.x;
    const int entry = sorted[p];
    uint8_t* d = dst + (size_t)p * row_bytes;
    if (entry < 0) {
        for (long o = (long)threadIdx.x * 16; o < row_bytes; o += (long)blockDim.x * 16)
            *reinterpret_cast<uint4*>(d + o) = make_uint4(0, 0, 0, 0);
        return;
    }
    const uint8_t* s = src + (size_t)(entry / top) * row_bytes;
    for (long o = (long)threadIdx.x * 16; o < row_bytes; o += (long)blockDim.x * 16)
        *reinterpret_cast<uint4*>(d + o) = *reinterpret_cast<const uint4*>(s + o);
}

// ------------------------------------------------------------------- the weighted sum
// sum[t, :] = sum_k weights[t, k] * (where[t * top + k] >= 0 ? y[where[t * top + k], :] : ident[t, :])  (+ gate[t] * shared[t, :])
// with k ascending, fp32: a pair that the sort left out (where < 0) belongs to an expert whose output is its input,
// `ident` [T, d] in Th.  Then out[t, :] = (accumulate ? out[t, :] : 0) + out_scale * (sum[t, :] + add[t, :]): `add` (fp32
// [T, d] or null) is what a sublayer beside the feed-forward made of the same x, and with `accumulate` the result goes
// straight into the residual stream.
template <typename Th>
__global__ void moe_combine_kernel(const float* __restrict__ y, long ldy, const int* __restrict__ where,
                                   const float* __restrict__ weights, int top, const float* __restrict__ shared,
                                   const float* __restrict__ gate, float* __restrict__ out, int d,
                                   const Th* __restrict__ ident, const float* __restrict__ add, float out_scale, int accumulate) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const bool plain = ident == nullptr && add == nullptr && out_scale == 1.0f && !accumulate;
    if (plain && d % 4 == 0 && ldy % 4 == 0 && ((((uintptr_t)y | (uintptr_t)shared | (uintptr_t)out) & 15) == 0)) {
        // four columns a thread (the same sums in the same order)
        for (int i = threadIdx.x * 4; i < d; i += blockDim.x * 4) {
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int k = 0; k < top; ++k) {
                const float wk = weights[(size_t)t * top + k];
                const float4 v = *reinterpret_cast<const float4*>(y + (size_t)where[(size_t)t * top + k] * ldy + i);
                acc.x = fmaf(wk, v.x, acc.x); acc.y = fmaf(wk, v.y, acc.y); acc.z = fmaf(wk, v.z, acc.z); acc.w = fmaf(wk, v.w, acc.w);
            }
            if (shared) {
                const float gt = gate ? gate[t] : 1.0f;
                const float4 v = *reinterpret_cast<const float4*>(shared + (size_t)t * d + i);
                acc.x = fmaf(gt, v.x, acc.x); acc.y = fmaf(gt, v.y, acc.y); acc.z = fmaf(gt, v.z, acc.z); acc.w = fmaf(gt, v.w, acc.w);
            }
            *reinterpret_cast<float4*>(out + (size_t)t * d + i) = acc;
        }
        return;
    }
    // The general form.  A token's rows and weights are looked up once (up to 8 choices in registers), then four columns a
    // thread and step where the rows allow it: the same sums in the same order as one column at a time.
    constexpr int MAXK = 8;
    int rows_k[MAXK];
    float w_k[MAXK];
    if (top <= MAXK) {
#pragma unroll
        for (int k = 0; k < MAXK; ++k) {
            rows_k[k] = k < top ? where[(size_t)t * top + k] : -1;
            w_k[k] = k < top ? weights[(size_t)t * top + k] : 0.f;
        }
    }
    const float gt = shared ? (gate ? gate[t] : 1.0f) : 0.f;
    const bool vec = top <= MAXK && d % 4 == 0 && ldy % 4 == 0 && sizeof(Th) == 4 &&
                     ((((uintptr_t)y | (uintptr_t)shared | (uintptr_t)out | (uintptr_t)add | (uintptr_t)ident) & 15) == 0);
    const bool vec_bf = top <= MAXK && d % 4 == 0 && ldy % 4 == 0 && sizeof(Th) == 2 &&
                        ((((uintptr_t)y | (uintptr_t)shared | (uintptr_t)out | (uintptr_t)add) & 15) == 0) && (((uintptr_t)ident & 7) == 0);
    if (vec || vec_bf) {
        for (int i = threadIdx.x * 4; i < d; i += blockDim.x * 4) {
            float4 idv = make_float4(0.f, 0.f, 0.f, 0.f);
            if (ident) {
                if (sizeof(Th) == 4) {
                    idv = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(ident) + (size_t)t * d + i);
                } else {
                    const uint2 u = *reinterpret_cast<const uint2*>(reinterpret_cast<const bf16*>(ident) + (size_t)t * d + i);
                    const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&u.x), hi = *reinterpret_cast<const __nv_bfloat162*>(&u.y);
                    idv = make_float4(__low2float(lo), __high2float(lo), __low2float(hi), __high2float(hi));
                }
            }
            float4 v[MAXK];
#pragma unroll
            for (int k = 0; k < MAXK; ++k)
                if (k < top) v[k] = rows_k[k] >= 0 ? *reinterpret_cast<const float4*>(y + (size_t)rows_k[k] * ldy + i) : idv;
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int k = 0; k < MAXK; ++k)
                if (k < top) {
                    acc.x = fmaf(w_k[k], v[k].x, acc.x); acc.y = fmaf(w_k[k], v[k].y, acc.y);
                    acc.z = fmaf(w_k[k], v[k].z, acc.z); acc.w = fmaf(w_k[k], v[k].w, acc.w);
                }
            if (shared) {
                const float4 sv = *reinterpret_cast<const float4*>(shared + (size_t)t * d + i);
                acc.x = fmaf(gt, sv.x, acc.x); acc.y = fmaf(gt, sv.y, acc.y); acc.z = fmaf(gt, sv.z, acc.z); acc.w = fmaf(gt, sv.w, acc.w);
            }
            if (add) {
                const float4 av = *reinterpret_cast<const float4*>(add + (size_t)t * d + i);
                acc.x += av.x; acc.y += av.y; acc.z += av.z; acc.w += av.w;
            }
            acc.x *= out_scale; acc.y *= out_scale; acc.z *= out_scale; acc.w *= out_scale;
            if (accumulate) {
                const float4 ov = *reinterpret_cast<const float4*>(out + (size_t)t * d + i);
                acc.x += ov.x; acc.y += ov.y; acc.z += ov.z; acc.w += ov.w;
            }
            *reinterpret_cast<float4*>(out + (size_t)t * d + i) = acc;
        }
        return;
    }
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float acc = 0.f;
        for (int k = 0; k < top; ++k) {
            const int row = where[(size_t)t * top + k];
            const float v = row >= 0 ? y[(size_t)row * ldy + i] : (ident ? to_f32<Th>(ident[(size_t)t * d + i]) : 0.f);
            acc = fmaf(weights[(size_t)t * top + k], v, acc);
        }
        if (shared) acc = fmaf(gate ? gate[t] : 1.0f, shared[(size_t)t * d + i], acc);
        if (add) acc += add[(size_t)t * d + i];
        acc *= out_scale;
        if (accumulate) acc += out[(size_t)t * d + i];
        out[(size_t)t * d + i] = acc;
    }
}

}  // namespace

// logits [T, E] fp32 = h [T, K] w [E, K]^T; h and w float32 or bfloat16 each.
extern "C" int plm_router_logits(const void* h, int h_dtype, const void* w, int w_dtype, float* out, int n_tokens, int E, int K,
                                 cudaStream_t stream) {
    if (n_tokens <= 0) return PLM_OK;
    if (E <= 0 || K <= 0) return PLM_ERR_SHAPE;
    const size_t smem = (size_t)RL_TOKENS * K * sizeof(float);
    if (smem > 200 * 1024) return PLM_ERR_SHAPE;
    const dim3 grid((n_tokens + RL_TOKENS - 1) / RL_TOKENS, (E + RL_WARPS - 1) / RL_WARPS), nt(RL_WARPS * 32);
#define RL_LAUNCH(Th_, Tw_)                                                                                            \
    do {                                                                                                               \
        if (smem > 48 * 1024)                                                                                          \
            cudaFuncSetAttribute(router_logits_kernel<Th_, Tw_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        return plm_status_of(launch_pdl(router_logits_kernel<Th_, Tw_>, grid, nt, smem, stream, (const Th_*)h, (const Tw_*)w, \
                                        out, n_tokens, E, K));                                                         \
    } while (0)
    if (h_dtype == PLM_F32 && w_dtype == PLM_F32) RL_LAUNCH(float, float);
    if (h_dtype == PLM_BF16 && w_dtype == PLM_BF16) RL_LAUNCH(bf16, bf16);
    if (h_dtype == PLM_BF16 && w_dtype == PLM_F32) RL_LAUNCH(bf16, float);
    if (h_dtype == PLM_F32 && w_dtype == PLM_BF16) RL_LAUNCH(float, bf16);
#undef RL_LAUNCH
    return PLM_ERR_DTYPE;
}

extern "C" int plm_route_topk(const float* logits, int ld, const float* correction, int E, int top, int n_groups,
                              int keep, float scale, int* ids, float* weights, float* gate, int gate_col, int n_tokens,
                              int softmax_scores, int group_by_max, int normalize, cudaStream_t stream) {
    if (n_tokens <= 0) return PLM_OK;
    if (E <= 0 || top <= 0 || top > E || n_groups <= 0 || E % n_groups || keep <= 0 || keep > n_groups || ld < E)
        return PLM_ERR_SHAPE;
    if (gate != nullptr && (gate_col < 0 || gate_col >= ld)) return PLM_ERR_SHAPE;
    const size_t smem = (size_t)ROUTE_WARPS * (2 * E + 2 * n_groups) * sizeof(float);
    if (smem > 200 * 1024) return PLM_ERR_SHAPE;
    if (smem > 48 * 1024) cudaFuncSetAttribute(route_topk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return plm_status_of(launch_pdl(route_topk_kernel, dim3((n_tokens + ROUTE_WARPS - 1) / ROUTE_WARPS), dim3(ROUTE_WARPS * 32),
                                    smem, stream, logits, ld, correction, E, top, n_groups, keep, scale, ids, weights, gate,
                                    gate_col, n_tokens, softmax_scores, group_by_max, normalize));
}

// The most tiles of `bm` rows that `n_entries` pairs over `n_experts` experts can fill: every tile holds at least
// one pair, and every expert leaves at most one tile part empty.
extern "C" int plm_moe_max_tiles(int n_entries, int n_experts, int bm) {
    const long a = ((long)n_entries + (long)n_experts * (bm - 1)) / bm;
    return (int)(a < n_entries ? a : n_entries);
}

extern "C" int plm_moe_align(const int* ids, int n_entries, int E, int bm, int* tile_expert, int* sorted, int* where,
                             int max_tiles, int n_skip, cudaStream_t stream) {
    if (n_entries <= 0) return PLM_OK;
    if (E <= 0 || bm <= 0 || max_tiles <= 0) return PLM_ERR_SHAPE;
    const size_t smem = (size_t)(3 * E + 1) * sizeof(int);
    if (smem > 200 * 1024) return PLM_ERR_SHAPE;
    if (smem > 48 * 1024) cudaFuncSetAttribute(moe_align_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return plm_status_of(launch_pdl(moe_align_kernel, dim3(1), dim3(ALIGN_NT), smem, stream, ids, n_entries, E, bm, tile_expert,
                                    sorted, where, max_tiles, n_skip));
}

// mode 0: gate/up with SiLU (a [T, K], out [max_tiles * bm, N] of a's type); mode 1: down (a [max_tiles * bm, K] of
// `dtype`, out fp32).  bm 16 or 64.  dtype: a and w, PLM_F32 or PLM_BF16.
// `interleaved` (mode 0): an expert's gate and up rows come in turns of 64 (64 gate rows, their 64 up rows, ...: the layout
// of the tensor-core product with the activation in its epilogue) instead of all gate rows before all up rows.
// bfloat16 with tiles of 16 rows, N a multiple of 8 and K of 32: the mma.sync kernel.
extern "C" int plm_moe_gemm(const void* a, long lda, int top, const void* w, void* out, long ldo, int dtype, int mode,
                            const int* tile_expert, const int* sorted, int max_tiles, int bm, int N, int K, int interleaved,
                            cudaStream_t stream) {
    if (max_tiles <= 0) return PLM_OK;
    if (N <= 0 || K <= 0 || top <= 0) return PLM_ERR_SHAPE;
    if (bm != 16 && bm != 64) return PLM_ERR_UNSUPPORTED;
    if (interleaved && (mode != 0 || N % 64)) return PLM_ERR_SHAPE;
    if (dtype == PLM_BF16 && bm == 16 && N % 8 == 0 && K % 32 == 0 && lda % 8 == 0 && ((((uintptr_t)a | (uintptr_t)w) & 15) == 0)) {
        const dim3 mgrid(max_tiles, (N + MM_BN - 1) / MM_BN), mnt(MM_WARPS * 32);
        const size_t smem = (size_t)16 * MM_LD * sizeof(bf16);
        if (mode == 0)
            return plm_status_of(launch_pdl(moe_gemm_mma_kernel<0>, mgrid, mnt, smem, stream, (const bf16*)a, lda, top, (const bf16*)w,
                                            out, ldo, tile_expert, sorted, N, K, interleaved));
        if (mode == 1)
            return plm_status_of(launch_pdl(moe_gemm_mma_kernel<1>, mgrid, mnt, smem, stream, (const bf16*)a, lda, top, (const bf16*)w,
                                            out, ldo, tile_expert, sorted, N, K, interleaved));
        return PLM_ERR_UNSUPPORTED;
    }
    const dim3 grid(max_tiles, (N + MG_BN - 1) / MG_BN), nt(256);
#define MG_LAUNCH(Ta_, To_, BM_, MODE_)                                                                              \
    return plm_status_of(launch_pdl(moe_gemm_kernel<Ta_, Ta_, To_, BM_, MODE_>, grid, nt, 0, stream, (const Ta_*)a, lda, top, \
                                    (const Ta_*)w, (To_*)out, ldo, tile_expert, sorted, N, K, interleaved))
    if (dtype == PLM_F32) {
        if (mode == 0) { if (bm == 16) MG_LAUNCH(float, float, 16, 0); else MG_LAUNCH(float, float, 64, 0); }
        if (mode == 1) { if (bm == 16) MG_LAUNCH(float, float, 16, 1); else MG_LAUNCH(float, float, 64, 1); }
    } else if (dtype == PLM_BF16) {
        if (mode == 0) { if (bm == 16) MG_LAUNCH(bf16, bf16, 16, 0); else MG_LAUNCH(bf16, bf16, 64, 0); }
        if (mode == 1) { if (bm == 16) MG_LAUNCH(bf16, float, 16, 1); else MG_LAUNCH(bf16, float, 64, 1); }
    } else {
        return PLM_ERR_DTYPE;
    }
#undef MG_LAUNCH
    return PLM_ERR_UNSUPPORTED;
}

extern "C" int plm_moe_gather(const void* src, void* dst, const int* sorted, int n_rows, int top, long row_bytes,
                              cudaStream_t stream) {
    if (n_rows <= 0) return PLM_OK;
    if (row_bytes <= 0 || row_bytes % 16 || (((uintptr_t)src | (uintptr_t)dst) & 15)) return PLM_ERR_ALIGN;
    return plm_status_of(launch_pdl(moe_gather_kernel, dim3(n_rows), dim3(128), 0, stream, (const uint8_t*)src, (uint8_t*)dst,
                                    sorted, top, row_bytes));
}

extern "C" int plm_moe_combine(const float* y, long ldy, const int* where, const float* weights, int top,
                               const float* shared, const float* gate, float* out, int n_tokens, int d, const void* ident,
                               int ident_dtype, const float* add, float out_scale, int accumulate, cudaStream_t stream) {
    if (n_tokens <= 0) return PLM_OK;
    if (d <= 0 || top <= 0) return PLM_ERR_SHAPE;
    if (ident != nullptr && ident_dtype == PLM_BF16)
        return plm_status_of(launch_pdl(moe_combine_kernel<bf16>, dim3(n_tokens), dim3(256), 0, stream, y, ldy, where, weights, top,
                                        shared, gate, out, d, (const bf16*)ident, add, out_scale, accumulate));
    if (ident != nullptr && ident_dtype != PLM_F32) return PLM_ERR_DTYPE;
    return plm_status_of(launch_pdl(moe_combine_kernel<float>, dim3(n_tokens), dim3(256), 0, stream, y, ldy, where, weights, top,
                                    shared, gate, out, d, (const float*)ident, add, out_scale, accumulate));
}
