// Kernels of the mixers that carry a fixed-size state from token to token, and of the small steps around
// them, for ragged steps (every sequence brings its own number of tokens, one in a decode step):
//
//   plm_causal_conv        depthwise causal convolution over the tokens of each sequence + SiLU, the last
//                          taps - 1 inputs of each sequence kept as state
//   plm_linear_scan        S_t = diag(d_t) S_(t-1) + k_t v_t^T, y_t = S_t^T q_t (+ skip * v_t): the recurrence
//                          of gated linear attention and of state-space duality, the decay per key channel
//                          or per head, computed from the raw projections inside the kernel in fp32
//   plm_gated_norm         grouped RMS norm with a multiplicative gate before or after it (or only one of the two)
//   plm_head_linear        out[t, h, :] = W[h] x[t, h, :]: one small matrix per head
//   plm_store_rows_paged   rows of the step's tokens into the pages of a cache
//
// Everything that enters a recurrence is fp32: decays, step sizes, the state, the sums.  T is the run's
// element type (float or bf16) of projections and activations; small parameter vectors are fp32.
#include "common.cuh"
#include <type_traits>

#define SCAN_THREADS 128
#define SCAN_PTILE 32

__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float log_sigmoid_f(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }
__device__ __forceinline__ float silu_f(float x) { return x / (1.f + expf(-x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + expf(-x)); }

// Two fp32 lanes in a 64-bit register; fma.rn.f32x2 rounds each lane as the scalar fma does.
__device__ __forceinline__ uint64_t pack2f(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(__float_as_uint(lo)), "r"(__float_as_uint(hi)));
    return r;
}
__device__ __forceinline__ void load8_bf16(const bf16* p, float* f) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        f[2 * e] = __low2float(h2[e]);
        f[2 * e + 1] = __high2float(h2[e]);
    }
}
__device__ __forceinline__ float lo2f(uint64_t v) { return __uint_as_float((uint32_t)v); }
__device__ __forceinline__ float hi2f(uint64_t v) { return __uint_as_float((uint32_t)(v >> 32)); }
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}

// ------------------------------------------------------------------------------------------------ convolution
// u [T, C] with row stride ldu; w [taps, C] (tap-major, so that neighbouring channels' weights are neighbours), the
// last tap being the current token's; state [slot][taps - 1][C], oldest first.  One block row per token, one thread
// per channel: inputs before the step's first token come from the state.
#define CONV_ACT_SILU 0
#define CONV_ACT_NONE 1
template <typename T>
__global__ void causal_conv_kernel(const T* __restrict__ u, long ldu, const float* __restrict__ w, const float* __restrict__ bias,
                                   const float* __restrict__ state, long state_stride, const int* __restrict__ tok_seq,
                                   const int* __restrict__ seq_start, const int* __restrict__ seq_slot, T* __restrict__ out,
                                   int n_tokens, int C, int taps, const float* __restrict__ in_bias, int act) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int b = PLM_SEQ_NO(tok_seq[t]);
    const int i = t - seq_start[b];
    const float* st = state + (long)seq_slot[b] * state_stride;
    float acc = bias ? bias[c] : 0.f;
    const float ib = in_bias ? in_bias[c] : 0.f;     // added to the step's inputs; the state holds inputs with it
    for (int j = 0; j < taps; ++j) {
        const int back = taps - 1 - j, li = i - back;
        const float val = li >= 0 ? to_f32<T>(u[(long)(t - back) * ldu + c]) + ib : st[(long)(taps - 1 + li) * C + c];
        acc = fmaf(w[(long)j * C + c], val, acc);
    }
    out[(long)t * C + c] = from_f32<T>(act == CONV_ACT_SILU ? silu_f(acc) : acc);
}

// The same for bf16 rows whose channels come in eights on 16-byte boundaries: a thread takes 8 channels of a token
// with one 16-byte load per tap.
__global__ void causal_conv_vec8_kernel(const bf16* __restrict__ u, long ldu, const float* __restrict__ w,
                                        const float* __restrict__ bias, const float* __restrict__ state, long state_stride,
                                        const int* __restrict__ tok_seq, const int* __restrict__ seq_start,
                                        const int* __restrict__ seq_slot, bf16* __restrict__ out, int n_tokens, int C, int taps) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x, c = (blockIdx.y * blockDim.x + threadIdx.x) << 3;
    if (c >= C) return;
    const int b = PLM_SEQ_NO(tok_seq[t]);
    const int i = t - seq_start[b];
    const float* st = state + (long)seq_slot[b] * state_stride;
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = bias ? bias[c + e] : 0.f;
    for (int j = 0; j < taps; ++j) {
        const int back = taps - 1 - j, li = i - back;
        float val[8];
        if (li >= 0) {
            const uint4 raw = *reinterpret_cast<const uint4*>(u + (long)(t - back) * ldu + c);
            const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                val[2 * e] = __low2float(h2[e]);
                val[2 * e + 1] = __high2float(h2[e]);
            }
        } else {
            const float* sr = st + (long)(taps - 1 + li) * C + c;
#pragma unroll
            for (int e = 0; e < 8; ++e) val[e] = sr[e];
        }
        const float4 w0 = *reinterpret_cast<const float4*>(w + (long)j * C + c), w1 = *reinterpret_cast<const float4*>(w + (long)j * C + c + 4);
        const float wr[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] = fmaf(wr[e], val[e], acc[e]);
    }
    __nv_bfloat162 o[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) o[e] = __floats2bfloat162_rn(silu_f(acc[2 * e]), silu_f(acc[2 * e + 1]));
    *reinterpret_cast<uint4*>(out + (long)t * C + c) = *reinterpret_cast<const uint4*>(o);
}

// The state after the step: the last taps - 1 inputs of old state followed by the step's tokens.  One thread per
// (sequence, channel); it reads what it needs of the old state before it writes.
template <typename T>
__global__ void causal_conv_state_kernel(const T* __restrict__ u, long ldu, float* __restrict__ state, long state_stride,
                                         const int* __restrict__ seq_start, const int* __restrict__ seq_slot, int n_seqs,
                                         int C, int taps, const float* __restrict__ in_bias) {
    pdl_launch_dependents();
    pdl_wait();
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long)n_seqs * C) return;
    const int b = (int)(idx / C), c = (int)(idx % C);
    const int t0 = seq_start[b], n = seq_start[b + 1] - t0;
    float* st = state + (long)seq_slot[b] * state_stride;
    // ascending s: slot s takes old slot s + n (> s), which no earlier iteration has overwritten
    for (int s = 0; s < taps - 1; ++s) {
        const int src = n - (taps - 1) + s;
        st[(long)s * C + c] = src >= 0 ? to_f32<T>(u[(long)(t0 + src) * ldu + c]) + (in_bias ? in_bias[c] : 0.f) : st[(long)(s + n) * C + c];
    }
}

// A decode step (one token per sequence): output and new state by the same thread.
template <typename T>
__global__ void causal_conv_decode_kernel(const T* __restrict__ u, long ldu, const float* __restrict__ w,
                                          const float* __restrict__ bias, float* __restrict__ state, long state_stride,
                                          const int* __restrict__ seq_slot, T* __restrict__ out, int n_seqs, int C, int taps,
                                          const float* __restrict__ in_bias, int act) {
    pdl_launch_dependents();
    pdl_wait();
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long)n_seqs * C) return;
    const int b = (int)(idx / C), c = (int)(idx % C);
    float* st = state + (long)seq_slot[b] * state_stride;
    const float cur = to_f32<T>(u[(long)b * ldu + c]) + (in_bias ? in_bias[c] : 0.f);
    float acc = bias ? bias[c] : 0.f;
    for (int j = 0; j < taps - 1; ++j) {
        const float val = st[(long)j * C + c];
        acc = fmaf(w[(long)j * C + c], val, acc);
        if (j > 0) st[(long)(j - 1) * C + c] = val;
    }
    acc = fmaf(w[(long)(taps - 1) * C + c], cur, acc);
    if (taps > 1) st[(long)(taps - 2) * C + c] = cur;
    out[(long)b * C + c] = from_f32<T>(act == CONV_ACT_SILU ? silu_f(acc) : acc);
}

extern "C" int plm_causal_conv(const void* u, int dtype, long ldu, const float* w, const float* bias, float* state,
                               long state_stride, const int* tok_seq, const int* seq_start, const int* seq_slot, void* out,
                               int n_tokens, int n_seqs, int C, int taps, int is_decode, const float* in_bias, int act,
                               cudaStream_t stream) {
    if (n_tokens <= 0 || n_seqs <= 0 || C <= 0 || taps < 1 || (act != CONV_ACT_SILU && act != CONV_ACT_NONE)) return PLM_ERR_SHAPE;
    if (dtype != PLM_F32 && dtype != PLM_BF16) return PLM_ERR_DTYPE;
    const int nt = 256;
    cudaError_t e;
    if (is_decode) {
        const unsigned grid = (unsigned)(((long)n_seqs * C + nt - 1) / nt);
        e = dtype == PLM_F32
                ? launch_pdl(causal_conv_decode_kernel<float>, dim3(grid), dim3(nt), 0, stream, (const float*)u, ldu, w, bias, state,
                             state_stride, seq_slot, (float*)out, n_seqs, C, taps, in_bias, act)
                : launch_pdl(causal_conv_decode_kernel<bf16>, dim3(grid), dim3(nt), 0, stream, (const bf16*)u, ldu, w, bias, state,
                             state_stride, seq_slot, (bf16*)out, n_seqs, C, taps, in_bias, act);
        return plm_status_of(e);
    }
    const dim3 grid((unsigned)n_tokens, (unsigned)((C + nt - 1) / nt));
    if (dtype == PLM_BF16 && in_bias == nullptr && act == CONV_ACT_SILU && C % 8 == 0 && ldu % 8 == 0 && (uintptr_t)u % 16 == 0 && (uintptr_t)out % 16 == 0 && (uintptr_t)w % 16 == 0)
        e = launch_pdl(causal_conv_vec8_kernel, dim3((unsigned)n_tokens, (unsigned)((C / 8 + 127) / 128)), dim3(128), 0, stream,
                       (const bf16*)u, ldu, w, bias, (const float*)state, state_stride, tok_seq, seq_start, seq_slot, (bf16*)out,
                       n_tokens, C, taps);
    else
    e = dtype == PLM_F32
            ? launch_pdl(causal_conv_kernel<float>, grid, dim3(nt), 0, stream, (const float*)u, ldu, w, bias, (const float*)state,
                         state_stride, tok_seq, seq_start, seq_slot, (float*)out, n_tokens, C, taps, in_bias, act)
            : launch_pdl(causal_conv_kernel<bf16>, grid, dim3(nt), 0, stream, (const bf16*)u, ldu, w, bias, (const float*)state,
                         state_stride, tok_seq, seq_start, seq_slot, (bf16*)out, n_tokens, C, taps, in_bias, act);
    if (e != cudaSuccess) return (int)e;
    if (taps == 1) return PLM_OK;
    const unsigned grid2 = (unsigned)(((long)n_seqs * C + nt - 1) / nt);
    e = dtype == PLM_F32
            ? launch_pdl(causal_conv_state_kernel<float>, dim3(grid2), dim3(nt), 0, stream, (const float*)u, ldu, state, state_stride,
                         seq_start, seq_slot, n_seqs, C, taps, in_bias)
            : launch_pdl(causal_conv_state_kernel<bf16>, dim3(grid2), dim3(nt), 0, stream, (const bf16*)u, ldu, state, state_stride,
                         seq_start, seq_slot, n_seqs, C, taps, in_bias);
    return plm_status_of(e);
}

// ------------------------------------------------------------------------------------------------ the scan
// How the decay d_t and the scale of v_t come out of the raw projections (all in fp32):
//   DECAY_STEP     per head: dt = softplus(raw[t, h] + p0[h]); d = exp(-exp(p1[h]) * dt); v_t is scaled by dt
//   DECAY_SIGMOID  per key channel: d[n] = exp(log_sigmoid(raw[t, h * N + n] + p0[h * N + n]) * power)
//   DECAY_GIVEN    per key channel, worked out beforehand: d[n] = raw[t, h * N + n], float32 (plm_sigmoid_decay
//                  makes these from the raw values where a step's tokens are walked twice)
#define DECAY_STEP 1
#define DECAY_SIGMOID 2
#define DECAY_GIVEN 3

// What a launch of the scan kernel does with the tokens of its segment:
//   SCAN_WHOLE  one segment per sequence: from the cache's state, writes y and the state (decode steps, short prompts)
//   SCAN_LOCAL  from zero, no y: leaves the segment's own contribution to the state and the product of its decays
//   SCAN_FINAL  from the state at the segment's start (put together by scan_combine_kernel), writes y; the last
//               segment of a sequence writes the cache's state
#define SCAN_WHOLE 0
#define SCAN_LOCAL 1
#define SCAN_FINAL 2

struct ScanArgs {
    const void *q, *k, *v, *raw;          // [T, groups * N], [T, groups * N], [T, H * P], the decay's raw values
    long ldq, ldk, ldv, ldraw;            // row strides in elements
    const float *p0, *p1, *skip;          // see the decay modes; skip[h] (or null): y += skip[h] * v_t (the unscaled v)
    float q_scale, power;
    float* state;                         // [slot][H][N][P]
    long state_stride;
    float* y;                             // [T, H * P]
    long ldy;
    const int *seq_start, *seq_slot;
    int n_seqs, H, N, P, heads_per_group;
    int seg_len, max_segs;                // tokens per segment; segments of the longest sequence
    float *seg_state, *seg_decay;         // [seq][segment][H][N][P] and [seq][segment][H][N]
    int vec8;                             // bf16 rows may be read eight channels at a time (sizes and addresses allow it)
};

// One block per (sequence, head, tile of 32 value columns, segment).  A warp holds 8 columns, two groups of 4; the
// N rows of a column group's state are dealt to 16 lanes (NS consecutive rows each), so a thread keeps NS x 4
// values of the state in registers.  The tokens are taken in order, TC at a time: the block first brings their q,
// k, decay and v to shared memory as fp32 (the exponentials are taken there, once per token and channel), then every
// thread steps its piece of the state through them; y's sum over the rows goes through the 16 lanes by shuffles.
template <typename T, int NS, int MODE, int PASS>
__global__ void __launch_bounds__(SCAN_THREADS, NS <= 8 ? 4 : 1) linear_scan_kernel(const ScanArgs a, int TC) {
    constexpr int ROW = NS == 4 ? 4 : NS + 4;             // padded so that a quarter warp's float4 reads hit different banks
    constexpr bool PER_CHANNEL = MODE != DECAY_STEP;
    extern __shared__ __align__(16) float smem[];
    pdl_launch_dependents();
    const int ptiles = (a.P + SCAN_PTILE - 1) / SCAN_PTILE;
    int bid = blockIdx.x;
    const int ptile = bid % ptiles;
    bid /= ptiles;
    const int h = bid % a.H, b = bid / a.H;
    const int seg = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int npart = lane & 15, pg = lane >> 4;
    const int pl = (warp << 3) + (pg << 2);               // first of this thread's 4 columns within the tile
    const int p = ptile * SCAN_PTILE + pl;
    const int g = h / a.heads_per_group;
    const int N = a.N, P = a.P;
    float* qs = smem;                                     // [TC][16][ROW]
    float* ks = qs + (long)TC * 16 * ROW;
    float* ds = ks + (long)TC * 16 * ROW;                 // per channel: [TC][16][ROW]; per head: [TC] decay, [TC] scale of v
    float* vs = ds + (PER_CHANNEL ? (long)TC * 16 * ROW : (long)((2 * TC + 3) & ~3));    // [TC][SCAN_PTILE]
    const T* q = (const T*)a.q;
    const T* k = (const T*)a.k;
    const T* v = (const T*)a.v;
    const T* raw = (const T*)a.raw;
    pdl_wait();
    const int s0 = a.seq_start[b], s1 = a.seq_start[b + 1];
    const int n_segs = PASS == SCAN_WHOLE ? 1 : (s1 - s0 + a.seg_len - 1) / a.seg_len;
    if (PASS == SCAN_LOCAL && seg >= n_segs - 1) return;  // nobody needs what the last segment adds by itself
    if (PASS == SCAN_FINAL && seg >= n_segs) return;
    const int t0 = PASS == SCAN_WHOLE ? s0 : s0 + seg * a.seg_len;
    const int t1 = PASS == SCAN_WHOLE ? s1 : min(s1, t0 + a.seg_len);
    float* st = a.state + (long)a.seq_slot[b] * a.state_stride + (long)h * N * P;
    float* sg = PASS == SCAN_WHOLE ? nullptr : a.seg_state + (((long)b * a.max_segs + seg) * a.H + h) * N * P;
    const float* init = PASS == SCAN_WHOLE ? st : PASS == SCAN_FINAL ? sg : nullptr;
    // The state in pairs of rows (2i, 2i + 1) of one column: the rows' k, q and decay lie side by side in shared
    // memory, so fma.rn.f32x2 takes them as they come and every instruction steps two elements of the state.
    uint64_t S[NS / 2][4];
    uint64_t dprod[PER_CHANNEL ? NS / 2 : 1];
    float dprod_h = 1.f;
#pragma unroll
    for (int i = 0; i < (PER_CHANNEL ? NS / 2 : 1); ++i) dprod[i] = pack2f(1.f, 1.f);
#pragma unroll
    for (int i = 0; i < NS / 2; ++i) {
        const int n = npart * NS + 2 * i;
#pragma unroll
        for (int j = 0; j < 4; ++j)
            S[i][j] = pack2f((init && n < N && p + j < P) ? init[(long)n * P + p + j] : 0.f,
                             (init && n + 1 < N && p + j < P) ? init[(long)(n + 1) * P + p + j] : 0.f);
    }
    const float skip = a.skip ? a.skip[h] : 0.f;
    // Rows of bf16 whose channels come in eights on 16-byte boundaries are brought in eight at a time (a.vec8, checked
    // by the host); the channels beyond N, which only pad the 16 lanes' shares, are filled once.
    const bool vec8 = sizeof(T) == 2 && a.vec8;
    if (vec8) {
        for (int idx = threadIdx.x; idx < TC * 16 * NS; idx += SCAN_THREADS) {
            const int tt = idx / (16 * NS), n = idx % (16 * NS);
            if (n < N) continue;
            const int at = (tt * 16 + n / NS) * ROW + n % NS;
            qs[at] = 0.f, ks[at] = 0.f;
            if (PER_CHANNEL) ds[at] = 1.f;
        }
    }
    for (int base = t0; base < t1; base += TC) {
        const int nt = min(TC, t1 - base);
        __syncthreads();
        if (vec8) {
            const int groups = N >> 3;
#pragma unroll 2
            for (int idx = threadIdx.x; idx < nt * groups; idx += SCAN_THREADS) {
                const int tt = idx / groups, n = (idx % groups) << 3;
                const int at = (tt * 16 + n / NS) * ROW + n % NS;
                const long row = base + tt;
                float f[8];
                if (PASS != SCAN_LOCAL) {
                    load8_bf16((const bf16*)q + row * a.ldq + (long)g * N + n, f);
                    *(float4*)(qs + at) = make_float4(f[0] * a.q_scale, f[1] * a.q_scale, f[2] * a.q_scale, f[3] * a.q_scale);
                    *(float4*)(qs + at + 4) = make_float4(f[4] * a.q_scale, f[5] * a.q_scale, f[6] * a.q_scale, f[7] * a.q_scale);
                }
                load8_bf16((const bf16*)k + row * a.ldk + (long)g * N + n, f);
                *(float4*)(ks + at) = make_float4(f[0], f[1], f[2], f[3]);
                *(float4*)(ks + at + 4) = make_float4(f[4], f[5], f[6], f[7]);
                if (MODE == DECAY_GIVEN) {
                    const float* dr = (const float*)a.raw + row * a.ldraw + (long)h * N + n;
                    *(float4*)(ds + at) = *(const float4*)dr;
                    *(float4*)(ds + at + 4) = *(const float4*)(dr + 4);
                }
                if (MODE == DECAY_SIGMOID) {
                    load8_bf16((const bf16*)raw + row * a.ldraw + (long)h * N + n, f);
                    const float* bias = a.p0 + (long)h * N + n;
#pragma unroll
                    for (int e = 0; e < 8; ++e) ds[at + e] = expf(log_sigmoid_f(f[e] + bias[e]) * a.power);
                }
            }
        } else {
#pragma unroll 8
            for (int idx = threadIdx.x; idx < nt * 16 * NS; idx += SCAN_THREADS) {
                const int tt = idx / (16 * NS), n = idx % (16 * NS);
                const int at = (tt * 16 + n / NS) * ROW + n % NS;
                const long row = base + tt;
                const bool in = n < N;
                if (PASS != SCAN_LOCAL) qs[at] = in ? to_f32<T>(q[row * a.ldq + (long)g * N + n]) * a.q_scale : 0.f;
                ks[at] = in ? to_f32<T>(k[row * a.ldk + (long)g * N + n]) : 0.f;
                if (MODE == DECAY_SIGMOID)
                    ds[at] = in ? expf(log_sigmoid_f(to_f32<T>(raw[row * a.ldraw + (long)h * N + n]) + a.p0[(long)h * N + n]) * a.power) : 1.f;
                if (MODE == DECAY_GIVEN) ds[at] = in ? ((const float*)a.raw)[row * a.ldraw + (long)h * N + n] : 1.f;
            }
        }
        if (!PER_CHANNEL) {
            for (int tt = threadIdx.x; tt < nt; tt += SCAN_THREADS) {
                const float dt = softplus_f(to_f32<T>(raw[(long)(base + tt) * a.ldraw + h]) + a.p0[h]);
                ds[tt] = expf(-expf(a.p1[h]) * dt);
                ds[TC + tt] = dt;
            }
        }
        if (vec8 && ptile * SCAN_PTILE + SCAN_PTILE <= P) {
            for (int idx = threadIdx.x; idx < nt * (SCAN_PTILE / 8); idx += SCAN_THREADS) {
                const int tt = idx / (SCAN_PTILE / 8), c = (idx % (SCAN_PTILE / 8)) << 3;
                float f[8];
                load8_bf16((const bf16*)v + (long)(base + tt) * a.ldv + (long)h * P + ptile * SCAN_PTILE + c, f);
                *(float4*)(vs + tt * SCAN_PTILE + c) = make_float4(f[0], f[1], f[2], f[3]);
                *(float4*)(vs + tt * SCAN_PTILE + c + 4) = make_float4(f[4], f[5], f[6], f[7]);
            }
        } else {
#pragma unroll 4
            for (int idx = threadIdx.x; idx < nt * SCAN_PTILE; idx += SCAN_THREADS) {
                const int tt = idx / SCAN_PTILE, c = idx % SCAN_PTILE, pc = ptile * SCAN_PTILE + c;
                vs[idx] = pc < P ? to_f32<T>(v[(long)(base + tt) * a.ldv + (long)h * P + pc]) : 0.f;
            }
        }
        __syncthreads();
        for (int tt = 0; tt < nt; ++tt) {
            const float4 x = *(const float4*)(vs + tt * SCAN_PTILE + pl);
            const float vsc = PER_CHANNEL ? 1.f : ds[TC + tt];
            const float4 vv = make_float4(vsc * x.x, vsc * x.y, vsc * x.z, vsc * x.w);
            const float dh = PER_CHANNEL ? 0.f : ds[tt];
            if (!PER_CHANNEL && PASS == SCAN_LOCAL) dprod_h *= dh;
            const uint64_t dh2 = pack2f(dh, dh), zero2 = 0ull;
            const uint64_t vv2[4] = {pack2f(vv.x, vv.x), pack2f(vv.y, vv.y), pack2f(vv.z, vv.z), pack2f(vv.w, vv.w)};
            const ulonglong2* q2 = (const ulonglong2*)(qs + (tt * 16 + npart) * ROW);
            const ulonglong2* k2 = (const ulonglong2*)(ks + (tt * 16 + npart) * ROW);
            const ulonglong2* d2 = (const ulonglong2*)(ds + (tt * 16 + npart) * ROW);
            uint64_t acc2[4] = {zero2, zero2, zero2, zero2};
#pragma unroll
            for (int i4 = 0; i4 < NS / 4; ++i4) {
                const ulonglong2 kk = k2[i4];
                ulonglong2 qq = make_ulonglong2(zero2, zero2), dd = make_ulonglong2(dh2, dh2);
                if (PASS != SCAN_LOCAL) qq = q2[i4];
                if (PER_CHANNEL) dd = d2[i4];
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    const uint64_t kp = half ? kk.y : kk.x, qp = half ? qq.y : qq.x, dp = half ? dd.y : dd.x;
                    uint64_t* Sr = S[2 * i4 + half];
                    if (PER_CHANNEL && PASS == SCAN_LOCAL) dprod[2 * i4 + half] = fma2(dprod[2 * i4 + half], dp, zero2);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        Sr[j] = fma2(dp, Sr[j], fma2(kp, vv2[j], zero2));
                        if (PASS != SCAN_LOCAL) acc2[j] = fma2(Sr[j], qp, acc2[j]);
                    }
                }
            }
            float4 acc;
            acc.x = lo2f(acc2[0]) + hi2f(acc2[0]);
            acc.y = lo2f(acc2[1]) + hi2f(acc2[1]);
            acc.z = lo2f(acc2[2]) + hi2f(acc2[2]);
            acc.w = lo2f(acc2[3]) + hi2f(acc2[3]);
            if (PASS != SCAN_LOCAL) {
                // Four sums over the 16 lanes in five shuffles: a lane gives away the half of its values that its
                // partner keeps (columns 0, 1 stay where bit 3 of the lane is clear, then one of the two where bit 2
                // is), after which lanes 0, 4, 8 and 12 of the group end up with the totals of columns 0, 1, 2, 3.
                const bool hi8 = npart & 8, hi4 = npart & 4;
                const float k0 = hi8 ? acc.z : acc.x, k1 = hi8 ? acc.w : acc.y;
                const float g0 = hi8 ? acc.x : acc.z, g1 = hi8 ? acc.y : acc.w;
                const float r0 = k0 + __shfl_xor_sync(0xffffffffu, g0, 8), r1 = k1 + __shfl_xor_sync(0xffffffffu, g1, 8);
                float tot = (hi4 ? r1 : r0) + __shfl_xor_sync(0xffffffffu, hi4 ? r0 : r1, 4);
                tot += __shfl_xor_sync(0xffffffffu, tot, 2);
                tot += __shfl_xor_sync(0xffffffffu, tot, 1);
                if ((npart & 3) == 0) {
                    const int j = npart >> 2;                 // which of the thread group's four columns this lane holds
                    const float xj = j == 0 ? x.x : j == 1 ? x.y : j == 2 ? x.z : x.w;
                    if (p + j < P) a.y[(long)(base + tt) * a.ldy + (long)h * P + p + j] = fmaf(skip, xj, tot);
                }
            }
        }
    }
    float* dst = PASS == SCAN_LOCAL ? sg : (PASS == SCAN_WHOLE || seg == n_segs - 1) ? st : nullptr;
    if (dst) {
#pragma unroll
        for (int i = 0; i < NS / 2; ++i) {
            const int n = npart * NS + 2 * i;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                if (n < N && p + j < P) dst[(long)n * P + p + j] = lo2f(S[i][j]);
                if (n + 1 < N && p + j < P) dst[(long)(n + 1) * P + p + j] = hi2f(S[i][j]);
            }
        }
    }
    if (PASS == SCAN_LOCAL && ptile == 0 && warp == 0 && pg == 0) {
        float* dd = a.seg_decay + (((long)b * a.max_segs + seg) * a.H + h) * N;
#pragma unroll
        for (int i = 0; i < NS; ++i) {
            const int n = npart * NS + i;
            const uint64_t pr = dprod[PER_CHANNEL ? i / 2 : 0];
            if (n < N) dd[n] = PER_CHANNEL ? ((i & 1) ? hi2f(pr) : lo2f(pr)) : dprod_h;
        }
    }
}

// Between the two passes over the segments: the state at the start of every segment, from the cache's state and
// what the segments before it add: S_in[0] = state, S_in[c + 1] = decay[c] * S_in[c] + local[c].  One thread per
// element of a sequence's state; S_in[c] takes local[c]'s place.
__global__ void scan_combine_kernel(const ScanArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    const long per_seq = (long)a.H * a.N * a.P;
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= per_seq * a.n_seqs) return;
    const int b = (int)(idx / per_seq);
    const long e = idx % per_seq;
    const long hn = e / a.P;
    const int n_segs = (a.seq_start[b + 1] - a.seq_start[b] + a.seg_len - 1) / a.seg_len;
    float S = a.state[(long)a.seq_slot[b] * a.state_stride + e];
    float* sg = a.seg_state + (long)b * a.max_segs * per_seq + e;
    const float* dd = a.seg_decay + (long)b * a.max_segs * a.H * a.N + hn;
    // eight segments' values are asked for at once, then chained
    for (int c0 = 0; c0 < n_segs; c0 += 8) {
        float local[8], decay[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int c = c0 + i;
            const bool more = c < n_segs - 1;
            local[i] = more ? sg[(long)c * per_seq] : 0.f;
            decay[i] = more ? dd[(long)c * a.H * a.N] : 0.f;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int c = c0 + i;
            if (c < n_segs) sg[(long)c * per_seq] = S;
            if (c < n_segs - 1) S = fmaf(decay[i], S, local[i]);
        }
    }
}

template <int NS>
static size_t scan_smem(int mode, int* TC) {
    const int ROW = NS == 4 ? 4 : NS + 4;
    // tokens per pass: as many as fit into about 40 KB of shared memory, 16 at most
    const long per_token = (mode != DECAY_STEP ? 3L : 2L) * 16 * ROW + SCAN_PTILE + (mode != DECAY_STEP ? 0 : 2);
    int tc = (int)((40 * 1024 / 4 - 4) / per_token);
    tc = tc > 16 ? 16 : tc < 1 ? 1 : tc;
    *TC = tc;
    return (size_t)(per_token * tc + 4) * sizeof(float);
}

template <typename T, int NS, int MODE>
static cudaError_t scan_launch(const ScanArgs& a, cudaStream_t stream) {
    int TC;
    const size_t smem = scan_smem<NS>(MODE, &TC);
    const int ptiles = (a.P + SCAN_PTILE - 1) / SCAN_PTILE;
    const unsigned blocks = (unsigned)((long)a.n_seqs * a.H * ptiles);
    if (a.max_segs <= 1)
        return launch_pdl(linear_scan_kernel<T, NS, MODE, SCAN_WHOLE>, dim3(blocks), dim3(SCAN_THREADS), smem, stream, a, TC);
    cudaError_t e = launch_pdl(linear_scan_kernel<T, NS, MODE, SCAN_LOCAL>, dim3(blocks, a.max_segs - 1), dim3(SCAN_THREADS), smem,
                               stream, a, TC);
    if (e != cudaSuccess) return e;
    const long elems = (long)a.n_seqs * a.H * a.N * a.P;
    e = launch_pdl(scan_combine_kernel, dim3((unsigned)((elems + 255) / 256)), dim3(256), 0, stream, a);
    if (e != cudaSuccess) return e;
    return launch_pdl(linear_scan_kernel<T, NS, MODE, SCAN_FINAL>, dim3(blocks, a.max_segs), dim3(SCAN_THREADS), smem, stream, a, TC);
}

template <typename T>
static int scan_dispatch(const ScanArgs& a, int mode, cudaStream_t stream) {
    const int ns = (a.N + 15) / 16;
    cudaError_t e;
#define SCAN_NS(NS_)                                                                       \
    (mode == DECAY_SIGMOID ? scan_launch<T, NS_, DECAY_SIGMOID>(a, stream)                 \
     : mode == DECAY_GIVEN ? scan_launch<T, NS_, DECAY_GIVEN>(a, stream)                   \
                           : scan_launch<T, NS_, DECAY_STEP>(a, stream))
    if (ns <= 4) e = SCAN_NS(4);
    else if (ns <= 8) e = SCAN_NS(8);
    else if (ns <= 16) e = SCAN_NS(16);
    else return PLM_ERR_UNSUPPORTED;
#undef SCAN_NS
    return plm_status_of(e);
}

// How a step of `n_tokens` tokens whose longest sequence brings `max_new` of them is cut: out[0] tokens per segment, out[1] segments of the
// longest sequence (1: one pass from the cache's state, no scratch memory).  Segments are worth their second pass
// when the sequences alone leave most of the GPU idle; there are as many as make one wave of blocks (a second, partly
// filled wave would take as long as the first), each of at least 64 tokens, and no more than keep the scratch memory
// under 1 GiB.
extern "C" int plm_linear_scan_plan(int n_seqs, int H, int N, int P, int max_new, int n_tokens, int* out) {
    out[0] = max_new > 0 ? max_new : 1;
    out[1] = 1;
    if (n_seqs <= 0 || H <= 0 || N <= 0 || P <= 0) return PLM_ERR_SHAPE;
    if (max_new < 192) return PLM_OK;
    // How many sequences' worth of work there is: the step's tokens over its longest sequence (a captured step
    // counts padding sequences without tokens among n_seqs, and a short sequence beside a long one fills few blocks).
    long busy = n_tokens > 0 ? ((long)n_tokens + max_new - 1) / max_new : n_seqs;
    if (busy > n_seqs) busy = n_seqs;
    if (busy < 1) busy = 1;
    const long blocks = busy * H * ((P + SCAN_PTILE - 1) / SCAN_PTILE);
    long segs = 4L * PLM_SM_COUNT / blocks;               // four blocks an SM run at once: one wave of them
    const long most = max_new / 64;
    if (segs > most) segs = most;
    const long state_bytes = (long)n_seqs * H * N * (P + 1) * 4;
    while (segs > 1 && segs * state_bytes > (1L << 30)) --segs;
    if (segs <= 1) return PLM_OK;
    int len = (int)((max_new + segs - 1) / segs);
    len = (len + 15) / 16 * 16;
    out[0] = len;
    out[1] = (max_new + len - 1) / len;
    return PLM_OK;
}

// out[t, c] = sigmoid(raw[t, c] + bias[c]) ^ power in fp32: the decays of DECAY_SIGMOID, worked out once.
template <typename T>
__global__ void sigmoid_decay_kernel(const T* __restrict__ raw, long ld, const float* __restrict__ bias, float power,
                                     float* __restrict__ out, int n_rows, int C) {
    pdl_launch_dependents();
    pdl_wait();
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long)n_rows * C) return;
    const long t = idx / C;
    const int c = (int)(idx % C);
    out[idx] = expf(log_sigmoid_f(to_f32<T>(raw[t * ld + c]) + bias[c]) * power);
}

extern "C" int plm_sigmoid_decay(const void* raw, int dtype, long ld, const float* bias, float power, float* out, int n_rows,
                                 int C, cudaStream_t stream) {
    if (n_rows <= 0 || C <= 0) return PLM_ERR_SHAPE;
    const unsigned grid = (unsigned)(((long)n_rows * C + 255) / 256);
    if (dtype == PLM_F32)
        return plm_status_of(launch_pdl(sigmoid_decay_kernel<float>, dim3(grid), dim3(256), 0, stream, (const float*)raw, ld, bias,
                                        power, out, n_rows, C));
    if (dtype == PLM_BF16)
        return plm_status_of(launch_pdl(sigmoid_decay_kernel<bf16>, dim3(grid), dim3(256), 0, stream, (const bf16*)raw, ld, bias,
                                        power, out, n_rows, C));
    return PLM_ERR_DTYPE;
}

extern "C" int plm_linear_scan(const void* q, const void* k, const void* v, const void* raw, int dtype, long ldq, long ldk,
                               long ldv, long ldraw, int mode, const float* p0, const float* p1, const float* skip,
                               float q_scale, float power, float* state, long state_stride, float* y, long ldy,
                               const int* seq_start, const int* seq_slot, int n_seqs, int H, int N, int P,
                               int heads_per_group, int seg_len, int max_segs, float* seg_state, float* seg_decay,
                               cudaStream_t stream) {
    if (n_seqs <= 0 || H <= 0 || N <= 0 || P <= 0 || heads_per_group <= 0) return PLM_ERR_SHAPE;
    if (mode != DECAY_STEP && mode != DECAY_SIGMOID && mode != DECAY_GIVEN) return PLM_ERR_UNSUPPORTED;
    if (mode == DECAY_STEP && !p1) return PLM_ERR_SHAPE;
    if (mode != DECAY_GIVEN && !p0) return PLM_ERR_SHAPE;
    if (N > 256) return PLM_ERR_UNSUPPORTED;
    if (max_segs > 1 && (!seg_state || !seg_decay || seg_len <= 0 || max_segs > 65535)) return PLM_ERR_SHAPE;
    ScanArgs a;
    a.q = q, a.k = k, a.v = v, a.raw = raw;
    a.ldq = ldq, a.ldk = ldk, a.ldv = ldv, a.ldraw = ldraw;
    a.p0 = p0, a.p1 = p1, a.skip = skip;
    a.q_scale = q_scale, a.power = power;
    a.state = state, a.state_stride = state_stride;
    a.y = y, a.ldy = ldy;
    a.seq_start = seq_start, a.seq_slot = seq_slot;
    a.n_seqs = n_seqs, a.H = H, a.N = N, a.P = P, a.heads_per_group = heads_per_group;
    a.seg_len = seg_len, a.max_segs = max_segs < 1 ? 1 : max_segs;
    a.seg_state = seg_state, a.seg_decay = seg_decay;
    const auto al = [](const void* p_, long ld, int bytes) { return (uintptr_t)p_ % 16 == 0 && (ld * bytes) % 16 == 0; };
    a.vec8 = dtype == PLM_BF16 && N % 8 == 0 && P % 8 == 0 && al(q, ldq, 2) && al(k, ldk, 2) && al(v, ldv, 2) &&
             (mode == DECAY_STEP || (mode == DECAY_GIVEN ? al(raw, ldraw, 4) : al(raw, ldraw, 2)));
    if (dtype == PLM_F32) return scan_dispatch<float>(a, mode, stream);
    if (dtype == PLM_BF16) return scan_dispatch<bf16>(a, mode, stream);
    return PLM_ERR_DTYPE;
}

// ------------------------------------------------------------------------------------------------ gate and norm
// One warp per (row, group of `group` consecutive columns):
//   val = x * act(gate)                       (gate_mode 1: the gate comes before the norm)
//   val = val / sqrt(mean(val^2) + eps) * w   (do_norm; w indexed by the column, or by the column within its group)
//   val = val * act(gate)                     (gate_mode 2: the gate comes after the norm)
// act: 0 SiLU, 1 sigmoid.  Statistics and products in fp32.
template <typename TI, typename TG, typename TO>
__global__ void gated_norm_kernel(const TI* __restrict__ x, long ldx, const TG* __restrict__ gate, long ldg,
                                  const float* __restrict__ w, int w_per_group, TO* __restrict__ out, long ldo, int n_rows,
                                  int C, int group, float eps, int gate_mode, int act, int do_norm) {
    pdl_launch_dependents();
    pdl_wait();
    const int groups = C / group;
    const long wid = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (wid >= (long)n_rows * groups) return;
    const long t = wid / groups;
    const int c0 = (int)(wid % groups) * group;
    const TI* xr = x + t * ldx + c0;
    const TG* gr = gate ? gate + t * ldg + c0 : nullptr;
    float r = 1.f;
    if (do_norm) {
        float ss = 0.f;
#pragma unroll 4
        for (int c = lane; c < group; c += 32) {
            float val = to_f32<TI>(xr[c]);
            if (gate_mode == 1) {
                const float gg = to_f32<TG>(gr[c]);
                val *= act ? sigmoid_f(gg) : silu_f(gg);
            }
            ss = fmaf(val, val, ss);
        }
        ss = warp_sum(ss);
        r = 1.f / sqrtf(ss / (float)group + eps);
    }
#pragma unroll 4
    for (int c = lane; c < group; c += 32) {
        float val = to_f32<TI>(xr[c]);
        float ga = 1.f;
        if (gate_mode) {
            const float gg = to_f32<TG>(gr[c]);
            ga = act ? sigmoid_f(gg) : silu_f(gg);
        }
        if (gate_mode == 1) val *= ga;
        if (do_norm) {
            val *= r;
            if (w) val *= w[w_per_group ? c : c0 + c];
        }
        if (gate_mode == 2) val *= ga;
        out[t * ldo + c0 + c] = from_f32<TO>(val);
    }
}

template <typename TI, typename TG, typename TO>
static int gated_norm_launch(const void* x, long ldx, const void* gate, long ldg, const float* w, int w_per_group, void* out,
                             long ldo, int n_rows, int C, int group, float eps, int gate_mode, int act, int do_norm,
                             cudaStream_t stream) {
    const long warps = (long)n_rows * (C / group);
    const unsigned grid = (unsigned)((warps * 32 + 255) / 256);
    return plm_status_of(launch_pdl(gated_norm_kernel<TI, TG, TO>, dim3(grid), dim3(256), 0, stream, (const TI*)x, ldx,
                                    (const TG*)gate, ldg, w, w_per_group, (TO*)out, ldo, n_rows, C, group, eps, gate_mode, act,
                                    do_norm));
}

extern "C" int plm_gated_norm(const void* x, int x_dtype, long ldx, const void* gate, int gate_dtype, long ldg, const float* w,
                              int w_per_group, void* out, int out_dtype, long ldo, int n_rows, int C, int group, float eps,
                              int gate_mode, int act, int do_norm, cudaStream_t stream) {
    if (n_rows <= 0 || C <= 0 || group <= 0 || C % group) return PLM_ERR_SHAPE;
    if (gate_mode && !gate) return PLM_ERR_SHAPE;
    if (!gate) gate_dtype = PLM_BF16;
    const int key = (x_dtype << 2) | (gate_dtype << 1) | out_dtype;
#define GN(TI, TG, TO) \
    return gated_norm_launch<TI, TG, TO>(x, ldx, gate, ldg, w, w_per_group, out, ldo, n_rows, C, group, eps, gate_mode, act, do_norm, stream)
    switch (key) {
        case (PLM_F32 << 2) | (PLM_F32 << 1) | PLM_F32: GN(float, float, float);
        case (PLM_F32 << 2) | (PLM_F32 << 1) | PLM_BF16: GN(float, float, bf16);
        case (PLM_F32 << 2) | (PLM_BF16 << 1) | PLM_F32: GN(float, bf16, float);
        case (PLM_F32 << 2) | (PLM_BF16 << 1) | PLM_BF16: GN(float, bf16, bf16);
        case (PLM_BF16 << 2) | (PLM_F32 << 1) | PLM_F32: GN(bf16, float, float);
        case (PLM_BF16 << 2) | (PLM_F32 << 1) | PLM_BF16: GN(bf16, float, bf16);
        case (PLM_BF16 << 2) | (PLM_BF16 << 1) | PLM_F32: GN(bf16, bf16, float);
        case (PLM_BF16 << 2) | (PLM_BF16 << 1) | PLM_BF16: GN(bf16, bf16, bf16);
    }
#undef GN
    return PLM_ERR_DTYPE;
}

// ------------------------------------------------------------------------------------------------ one matrix per head
// out[t, h, o] = sum_i W[h][o][i] * x[t, h, i], optionally times sigmoid(gate[t, h, o]) (gate_per_head: one gate a head,
// sigmoid(gate[t, h])).  x [T, H * I] with row stride ldx, W [H, O, I], out [T, H * O].  Tiles of 64 tokens x 64 outputs, 4 x 4 of them a thread, the inputs walked 32 at
// a time through shared memory, sums in fp32 in ascending order of i.
#define HL_TT 64
#define HL_TO 64
#define HL_TI 32
template <typename T, typename TG>
__global__ void __launch_bounds__(256) head_linear_kernel(const T* __restrict__ x, long ldx, const T* __restrict__ W,
                                                          const TG* __restrict__ gate, long ldg, T* __restrict__ out, long ldo,
                                                          int n_tokens, int H, int O, int I, int gate_per_head) {
    __shared__ float xs[HL_TI][HL_TT + 4];                 // transposed: a thread reads its 4 tokens as one float4
    __shared__ float ws[HL_TI][HL_TO + 4];
    pdl_launch_dependents();
    const int h = blockIdx.z, t0 = blockIdx.y * HL_TT, o0 = blockIdx.x * HL_TO;
    const int og = threadIdx.x % 16, tg = threadIdx.x / 16;               // 4 outputs x 4 tokens a thread
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    pdl_wait();
    for (int i0 = 0; i0 < I; i0 += HL_TI) {
        __syncthreads();
        for (int idx = threadIdx.x; idx < HL_TT * HL_TI; idx += 256) {
            const int tt = idx / HL_TI, ii = idx % HL_TI;
            xs[ii][tt] = (t0 + tt < n_tokens && i0 + ii < I) ? to_f32<T>(x[(long)(t0 + tt) * ldx + (long)h * I + i0 + ii]) : 0.f;
        }
        for (int idx = threadIdx.x; idx < HL_TO * HL_TI; idx += 256) {
            const int oo = idx / HL_TI, ii = idx % HL_TI;
            ws[ii][oo] = (o0 + oo < O && i0 + ii < I) ? to_f32<T>(W[((long)h * O + o0 + oo) * I + i0 + ii]) : 0.f;
        }
        __syncthreads();
#pragma unroll 8
        for (int ii = 0; ii < HL_TI; ++ii) {
            const float4 xv = *(const float4*)&xs[ii][tg * 4];
            const float4 wv = *(const float4*)&ws[ii][og * 4];
            const float xr[4] = {xv.x, xv.y, xv.z, xv.w}, wr[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(wr[j], xr[i], acc[i][j]);
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int t = t0 + tg * 4 + i;
        if (t >= n_tokens) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int o = o0 + og * 4 + j;
            if (o >= O) continue;
            float val = acc[i][j];
            if (gate) val *= sigmoid_f(to_f32<TG>(gate[(long)t * ldg + (gate_per_head ? (long)h : (long)h * O + o)]));
            out[(long)t * ldo + (long)h * O + o] = from_f32<T>(val);
        }
    }
}

// The same for a handful of tokens (a decode step): the weights are what has to be read, once.  One warp per output
// row (h, o): it takes the row's I weights into registers (up to 32 a lane) and forms the dot product with every
// token's x[t, h, :]; a lane's elements are I / 32 apart so that the warp's loads are contiguous.
#define HLS_MAX_T 16
template <typename T, typename TG>
__global__ void __launch_bounds__(256) head_linear_small_kernel(const T* __restrict__ x, long ldx, const T* __restrict__ W,
                                                                const TG* __restrict__ gate, long ldg, T* __restrict__ out,
                                                                long ldo, int n_tokens, int H, int O, int I, int gate_per_head) {
    pdl_launch_dependents();
    const long row = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;          // h * O + o
    const int lane = threadIdx.x & 31;
    if (row >= (long)H * O) return;
    const int h = (int)(row / O);
    float wr[32];
    const T* wp = W + row * I;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
        const int c = lane + 32 * i;
        wr[i] = c < I ? to_f32<T>(wp[c]) : 0.f;
    }
    pdl_wait();
    for (int t = 0; t < n_tokens; ++t) {
        const T* xr = x + (long)t * ldx + (long)h * I;
        float acc = 0.f;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            const int c = lane + 32 * i;
            if (c < I) acc = fmaf(wr[i], to_f32<T>(xr[c]), acc);
        }
        acc = warp_sum(acc);
        if (lane == 0) {
            if (gate) acc *= sigmoid_f(to_f32<TG>(gate[(long)t * ldg + (gate_per_head ? (long)h : row)]));
            out[(long)t * ldo + row] = from_f32<T>(acc);
        }
    }
}

template <typename T, typename TG>
static int head_linear_launch(const void* x, long ldx, const void* W, const void* gate, long ldg, void* out, long ldo, int n_tokens,
                              int H, int O, int I, int gate_per_head, cudaStream_t stream) {
    if (n_tokens <= HLS_MAX_T && I <= 1024) {
        const unsigned blocks = (unsigned)(((long)H * O * 32 + 255) / 256);
        return plm_status_of(launch_pdl(head_linear_small_kernel<T, TG>, dim3(blocks), dim3(256), 0, stream, (const T*)x, ldx,
                                        (const T*)W, (const TG*)gate, ldg, (T*)out, ldo, n_tokens, H, O, I, gate_per_head));
    }
    const dim3 grid((O + HL_TO - 1) / HL_TO, (n_tokens + HL_TT - 1) / HL_TT, H);
    if (grid.y > 65535) return PLM_ERR_SHAPE;
    return plm_status_of(launch_pdl(head_linear_kernel<T, TG>, grid, dim3(256), 0, stream, (const T*)x, ldx, (const T*)W,
                                    (const TG*)gate, ldg, (T*)out, ldo, n_tokens, H, O, I, gate_per_head));
}

// dtype: x, W and out; gate_dtype: the gate (that type or PLM_F32)
extern "C" int plm_head_linear(const void* x, int dtype, long ldx, const void* W, const void* gate, int gate_dtype, long ldg,
                               void* out, long ldo, int n_tokens, int H, int O, int I, int gate_per_head, cudaStream_t stream) {
    if (n_tokens <= 0 || H <= 0 || O <= 0 || I <= 0 || H > 65535) return PLM_ERR_SHAPE;
    if (gate == nullptr) gate_dtype = dtype;
    if (dtype == PLM_F32 && gate_dtype == PLM_F32)
        return head_linear_launch<float, float>(x, ldx, W, gate, ldg, out, ldo, n_tokens, H, O, I, gate_per_head, stream);
    if (dtype == PLM_BF16 && gate_dtype == PLM_BF16)
        return head_linear_launch<bf16, bf16>(x, ldx, W, gate, ldg, out, ldo, n_tokens, H, O, I, gate_per_head, stream);
    if (dtype == PLM_BF16 && gate_dtype == PLM_F32)
        return head_linear_launch<bf16, float>(x, ldx, W, gate, ldg, out, ldo, n_tokens, H, O, I, gate_per_head, stream);
    return PLM_ERR_DTYPE;
}

// ------------------------------------------------------------------------------------------------ rows into pages
// pages [n_pages][PLM_PAGE][R] (one kv head): row t goes to position tok_pos[t] of sequence tok_seq[t].
template <typename T>
__global__ void store_rows_paged_kernel(const T* __restrict__ rows, long ld, T* __restrict__ pages, const int* __restrict__ tok_pos,
                                        const int* __restrict__ tok_seq, const int* __restrict__ block_table, int pages_per_seq,
                                        int n_tokens, int R) {
    pdl_launch_dependents();
    pdl_wait();
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long)n_tokens * R) return;
    const int t = (int)(idx / R), c = (int)(idx % R);
    const int pos = PLM_POSITION(tok_pos[t]);
    const int page = PLM_PAGE_NO(block_table[(long)PLM_SEQ_NO(tok_seq[t]) * pages_per_seq + pos / PLM_PAGE]);
    pages[((long)page * PLM_PAGE + pos % PLM_PAGE) * R + c] = rows[(long)t * ld + c];
}

extern "C" int plm_store_rows_paged(const void* rows, int dtype, long ld, void* pages, const int* tok_pos, const int* tok_seq,
                                    const int* block_table, int pages_per_seq, int n_tokens, int R, cudaStream_t stream) {
    if (n_tokens <= 0 || R <= 0) return PLM_ERR_SHAPE;
    const unsigned grid = (unsigned)(((long)n_tokens * R + 255) / 256);
    cudaError_t e;
    if (dtype == PLM_F32)
        e = launch_pdl(store_rows_paged_kernel<float>, dim3(grid), dim3(256), 0, stream, (const float*)rows, ld, (float*)pages, tok_pos,
                       tok_seq, block_table, pages_per_seq, n_tokens, R);
    else if (dtype == PLM_BF16)
        e = launch_pdl(store_rows_paged_kernel<bf16>, dim3(grid), dim3(256), 0, stream, (const bf16*)rows, ld, (bf16*)pages, tok_pos,
                       tok_seq, block_table, pages_per_seq, n_tokens, R);
    else
        return PLM_ERR_DTYPE;
    return plm_status_of(e);
}

// A latent's row as the cache keeps it, made from the projection's columns in one pass: rows [T, n_rot + n_norm] with row
// stride ld hold `n_rot` columns that are rotated by the token's position (half-split or neighbouring pairs; a key part
// that all heads share) and then `n_norm` columns that are divided by their root mean square (eps inside the root) and
// multiplied by w [n_norm] (fp32); the page's row is [rotated | normed | zeros] of width R >= n_rot + n_norm.  Everything
// in fp32; one warp per token, the sum of squares in an order that depends on n_norm only.  The same warp can norm a second
// stretch of the token's row on the way (the queries' latent, which the same product made): q_rows [T, n_q] with stride
// ldq, divided by their root mean square and multiplied by wq [n_q], to q_out [T, n_q] (contiguous).
template <typename Ti, typename To>
__global__ void __launch_bounds__(128)
latent_store_kernel(const Ti* __restrict__ rows, long ld, const float* __restrict__ w, float eps, const float* __restrict__ cos_t,
                    const float* __restrict__ sin_t, To* __restrict__ pages, const int* __restrict__ tok_pos,
                    const int* __restrict__ tok_seq, const int* __restrict__ block_table, int pages_per_seq, int n_tokens,
                    int n_rot, int n_norm, int R, int pairing, int store, const Ti* __restrict__ q_rows, long ldq,
                    const float* __restrict__ wq, To* __restrict__ q_out, int n_q) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (t >= n_tokens) return;
    if (q_rows) {
        const Ti* qs = q_rows + (long)t * ldq;
        float sq = 0.f;
        for (int j = lane; j < n_q; j += 32) {
            const float v = to_f32<Ti>(qs[j]);
            sq = fmaf(v, v, sq);
        }
        const float rq = 1.0f / sqrtf(warp_sum(sq) / (float)n_q + eps);
        for (int j = lane; j < n_q; j += 32) q_out[(long)t * n_q + j] = from_f32<To>(to_f32<Ti>(qs[j]) * rq * wq[j]);
    }
    if (!store) return;
    const int pos = PLM_POSITION(tok_pos[t]);
    const int page = PLM_PAGE_NO(block_table[(long)PLM_SEQ_NO(tok_seq[t]) * pages_per_seq + pos / PLM_PAGE]);
    const Ti* src = rows + (long)t * ld;
    To* dst = pages + ((long)page * PLM_PAGE + pos % PLM_PAGE) * R;
    float ss = 0.f;
    for (int j = lane; j < n_norm; j += 32) {
        const float v = to_f32<Ti>(src[n_rot + j]);
        ss = fmaf(v, v, ss);
    }
    const float r = 1.0f / sqrtf(warp_sum(ss) / (float)n_norm + eps);
    const int half = n_rot / 2;
    for (int j = lane; j < half; j += 32) {
        const int ia = pairing == 0 ? j : 2 * j, ib = pairing == 0 ? j + half : 2 * j + 1;
        const float a = to_f32<Ti>(src[ia]), b = to_f32<Ti>(src[ib]);
        const float c = cos_t[(size_t)pos * half + j], s = sin_t[(size_t)pos * half + j];
        dst[ia] = from_f32<To>(__fsub_rn(__fmul_rn(a, c), __fmul_rn(b, s)));
        dst[ib] = from_f32<To>(__fadd_rn(__fmul_rn(a, s), __fmul_rn(b, c)));
    }
    for (int j = lane; j < n_norm; j += 32) dst[n_rot + j] = from_f32<To>(to_f32<Ti>(src[n_rot + j]) * r * w[j]);
    for (int j = n_rot + n_norm + lane; j < R; j += 32) dst[j] = from_f32<To>(0.f);
}

extern "C" int plm_latent_store(const void* rows, int in_dtype, long ld, const float* w, float eps, const float* cos_t,
                                const float* sin_t, void* pages, int out_dtype, const int* tok_pos, const int* tok_seq,
                                const int* block_table, int pages_per_seq, int n_tokens, int n_rot, int n_norm, int R,
                                int pairing, int store, const void* q_rows, long ldq, const float* wq, void* q_out, int n_q,
                                cudaStream_t stream) {
    if (n_tokens <= 0) return PLM_OK;
    if (n_rot < 0 || (n_rot & 1) || n_norm <= 0 || R < n_rot + n_norm || ld < n_rot + n_norm || (n_rot > 0 && cos_t == nullptr))
        return PLM_ERR_SHAPE;
    if (q_rows != nullptr && (n_q <= 0 || ldq < n_q || wq == nullptr || q_out == nullptr)) return PLM_ERR_SHAPE;
    if (!store && q_rows == nullptr) return PLM_OK;
    if (pairing != 0 && pairing != 1) return PLM_ERR_UNSUPPORTED;
    const dim3 grid((unsigned)((n_tokens + 3) / 4));
#define LS_LAUNCH(Ti_, To_)                                                                                                     \
    return plm_status_of(launch_pdl(latent_store_kernel<Ti_, To_>, grid, dim3(128), 0, stream, (const Ti_*)rows, ld, w, eps, cos_t, \
                                    sin_t, (To_*)pages, tok_pos, tok_seq, block_table, pages_per_seq, n_tokens, n_rot, n_norm, R, \
                                    pairing, store, (const Ti_*)q_rows, ldq, wq, (To_*)q_out, n_q))
    if (in_dtype == PLM_F32 && out_dtype == PLM_F32) LS_LAUNCH(float, float);
    if (in_dtype == PLM_F32 && out_dtype == PLM_BF16) LS_LAUNCH(float, bf16);
    if (in_dtype == PLM_BF16 && out_dtype == PLM_BF16) LS_LAUNCH(bf16, bf16);
#undef LS_LAUNCH
    return PLM_ERR_DTYPE;
}

// ------------------------------------------------------------------------------------------------ gated diagonal recurrence
// The real-gated linear recurrent unit: the channels come in `B` blocks of n; in block b
//   zr = Wr[b] u_b + br,  zi = Wi[b] u_b + bi   (Wr[b], Wi[b] square, [out, in])
//   log a = -sigmoid(zr) * rate,  a = exp(log a),  x = sqrt(1 - a^2) * sigmoid(zi) * u
// with rate = 8 softplus(lambda) worked out once by the host.  1 - a^2 is taken as -expm1(2 log a), which keeps its
// digits where a is close to 1, and what is handed on is log a, not a: a float next to 1 has lost the digits of
// 1 - a, on which a state that lasts thousands of tokens depends.  The sums are fp32 and run over k in ascending order for every element; with float32
// inputs each piece of 32 terms is folded into a double (a decay close to 1 multiplies what its gate's sum loses).
// One block: 32 tokens x 32 channels of one gate block, K in pieces of 32 through shared memory.
__device__ __forceinline__ float gelu_tanh_f(float z) {
    return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

template <typename T, typename Tw>
__global__ void __launch_bounds__(256)
rglru_gates_kernel(const T* __restrict__ u, long ldu, const Tw* __restrict__ wr, const Tw* __restrict__ wi,
                   const float* __restrict__ br, const float* __restrict__ bi, const float* __restrict__ rate,
                   float* __restrict__ a_out, float* __restrict__ x_out, int n_tokens, int W, int n) {
    __shared__ float us[32][33], wrs[32][33], wis[32][33];
    pdl_launch_dependents();
    pdl_wait();
    const int t0 = blockIdx.x * 32, blk = blockIdx.y, o0 = blockIdx.z * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    constexpr bool kWide = std::is_same<T, float>::value;
    float zr[4] = {0.f, 0.f, 0.f, 0.f}, zi[4] = {0.f, 0.f, 0.f, 0.f};
    double zr_w[4] = {0.0, 0.0, 0.0, 0.0}, zi_w[4] = {0.0, 0.0, 0.0, 0.0};
    for (int k0 = 0; k0 < n; k0 += 32) {
        const int kk = k0 + tx;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int row = ty + 8 * j, tt = t0 + row, oo = o0 + row;
            us[row][tx] = (tt < n_tokens && kk < n) ? to_f32<T>(u[(long)tt * ldu + (long)blk * n + kk]) : 0.f;
            const bool in = oo < n && kk < n;
            const long at = ((long)blk * n + oo) * n + kk;
            wrs[row][tx] = in ? to_f32<Tw>(wr[at]) : 0.f;
            wis[row][tx] = in ? to_f32<Tw>(wi[at]) : 0.f;
        }
        __syncthreads();
#pragma unroll 8
        for (int k = 0; k < 32; ++k) {
            const float a = wrs[tx][k], b = wis[tx][k];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float uv = us[ty + 8 * j][k];
                zr[j] = fmaf(a, uv, zr[j]);
                zi[j] = fmaf(b, uv, zi[j]);
            }
        }
        if (kWide) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                zr_w[j] += (double)zr[j], zi_w[j] += (double)zi[j];
                zr[j] = zi[j] = 0.f;
            }
        }
        __syncthreads();
    }
    if (kWide) {
#pragma unroll
        for (int j = 0; j < 4; ++j) zr[j] = (float)zr_w[j], zi[j] = (float)zi_w[j];
    }
    const int o = o0 + tx;
    if (o >= n) return;
    const int c = blk * n + o;
    const float b_r = br[c], b_i = bi[c], rt = rate[c];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int tt = t0 + ty + 8 * j;
        if (tt >= n_tokens) continue;
        const float uu = to_f32<T>(u[(long)tt * ldu + c]);
        const float la = -sigmoid_f(zr[j] + b_r) * rt;
        a_out[(long)tt * W + c] = la;
        x_out[(long)tt * W + c] = sqrtf(-expm1f(2.f * la)) * sigmoid_f(zi[j] + b_i) * uu;
    }
}

extern "C" int plm_rglru_gates(const void* u, int dtype, long ldu, const void* wr, const void* wi, int w_dtype, const float* br,
                               const float* bi, const float* rate, float* a_out, float* x_out, int n_tokens, int W, int blocks,
                               cudaStream_t stream) {
    if (n_tokens <= 0) return PLM_OK;
    if (W <= 0 || blocks <= 0 || W % blocks) return PLM_ERR_SHAPE;
    const int n = W / blocks;
    const dim3 grid((unsigned)((n_tokens + 31) / 32), (unsigned)blocks, (unsigned)((n + 31) / 32));
    if (dtype == PLM_F32 && w_dtype == PLM_F32)
        return plm_status_of(launch_pdl(rglru_gates_kernel<float, float>, grid, dim3(256), 0, stream, (const float*)u, ldu,
                                        (const float*)wr, (const float*)wi, br, bi, rate, a_out, x_out, n_tokens, W, n));
    if (dtype == PLM_BF16 && w_dtype == PLM_BF16)
        return plm_status_of(launch_pdl(rglru_gates_kernel<bf16, bf16>, grid, dim3(256), 0, stream, (const bf16*)u, ldu,
                                        (const bf16*)wr, (const bf16*)wi, br, bi, rate, a_out, x_out, n_tokens, W, n));
    return PLM_ERR_DTYPE;
}

// S_t = a_t S_(t-1) + x_t per channel over each sequence's tokens, out_t = S_t * gelu_tanh(y_t + y_bias), with a_t given
// as its logarithm.  a_t is taken as 1 + expm1(log a_t) in double and S is walked in double, so that neither a decay
// next to 1 nor a long prompt loses digits; the state is kept in the cache as float32.  One block
// per (32 channels, sequence): its 32 warps take 32 equal stretches of the sequence's tokens; a first walk leaves each
// stretch's product of decays and its own sum, one warp chains them from the cache's state, a second walk writes.
template <typename T>
__global__ void __launch_bounds__(1024)
diag_scan_kernel(const float* __restrict__ a, const float* __restrict__ x, const T* __restrict__ yraw, long ldy,
                 const float* __restrict__ ybias, float* __restrict__ state, long state_stride, T* __restrict__ out,
                 const int* __restrict__ seq_start, const int* __restrict__ seq_slot, int W) {
    __shared__ double As[32][33], Bs[32][33];
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.y, lane = threadIdx.x & 31, seg = threadIdx.x >> 5;
    const int c = blockIdx.x * 32 + lane;
    const int s0 = seq_start[b], s1 = seq_start[b + 1];
    if (s1 <= s0) return;
    const int L = (s1 - s0 + 31) / 32;
    const int t0 = min(s1, s0 + seg * L), t1 = min(s1, t0 + L);
    double A = 1.0, Bv = 0.0;
    if (c < W)
        for (int t = t0; t < t1; ++t) {
            const double av = 1.0 + (double)expm1f(a[(long)t * W + c]);
            Bv = fma(av, Bv, (double)x[(long)t * W + c]);
            A *= av;
        }
    As[seg][lane] = A;
    Bs[seg][lane] = Bv;
    __syncthreads();
    if (seg == 0 && c < W) {
        float* st = state + (long)seq_slot[b] * state_stride;
        double carry = (double)st[c];
        for (int s = 0; s < 32; ++s) {
            const double sa = As[s][lane], sb = Bs[s][lane];
            As[s][lane] = carry;
            carry = fma(sa, carry, sb);
        }
        st[c] = (float)carry;
    }
    __syncthreads();
    if (c >= W) return;
    double S = As[seg][lane];
    const float yb = ybias ? ybias[c] : 0.f;
    for (int t = t0; t < t1; ++t) {
        S = fma(1.0 + (double)expm1f(a[(long)t * W + c]), S, (double)x[(long)t * W + c]);
        out[(long)t * W + c] = from_f32<T>((float)S * gelu_tanh_f(to_f32<T>(yraw[(long)t * ldy + c]) + yb));
    }
}

// A decode step: one token per sequence, one thread per (sequence, channel).
template <typename T>
__global__ void diag_scan_decode_kernel(const float* __restrict__ a, const float* __restrict__ x, const T* __restrict__ yraw,
                                        long ldy, const float* __restrict__ ybias, float* __restrict__ state, long state_stride,
                                        T* __restrict__ out, const int* __restrict__ seq_slot, int n_seqs, int W) {
    pdl_launch_dependents();
    pdl_wait();
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long)n_seqs * W) return;
    const int b = (int)(idx / W), c = (int)(idx % W);
    float* st = state + (long)seq_slot[b] * state_stride;
    const float S = (float)fma(1.0 + (double)expm1f(a[idx]), (double)st[c], (double)x[idx]);
    st[c] = S;
    out[idx] = from_f32<T>(S * gelu_tanh_f(to_f32<T>(yraw[(long)b * ldy + c]) + (ybias ? ybias[c] : 0.f)));
}

extern "C" int plm_diag_scan(const float* a, const float* x, const void* yraw, int dtype, long ldy, const float* ybias,
                             float* state, long state_stride, void* out, const int* seq_start, const int* seq_slot, int n_seqs,
                             int W, int is_decode, cudaStream_t stream) {
    if (n_seqs <= 0) return PLM_OK;
    if (W <= 0) return PLM_ERR_SHAPE;
    if (dtype != PLM_F32 && dtype != PLM_BF16) return PLM_ERR_DTYPE;
    if (is_decode) {
        const dim3 grid((unsigned)(((long)n_seqs * W + 255) / 256));
        return plm_status_of(dtype == PLM_F32
            ? launch_pdl(diag_scan_decode_kernel<float>, grid, dim3(256), 0, stream, a, x, (const float*)yraw, ldy, ybias, state,
                         state_stride, (float*)out, seq_slot, n_seqs, W)
            : launch_pdl(diag_scan_decode_kernel<bf16>, grid, dim3(256), 0, stream, a, x, (const bf16*)yraw, ldy, ybias, state,
                         state_stride, (bf16*)out, seq_slot, n_seqs, W));
    }
    const dim3 grid((unsigned)((W + 31) / 32), (unsigned)n_seqs);
    return plm_status_of(dtype == PLM_F32
        ? launch_pdl(diag_scan_kernel<float>, grid, dim3(1024), 0, stream, a, x, (const float*)yraw, ldy, ybias, state, state_stride,
                     (float*)out, seq_start, seq_slot, W)
        : launch_pdl(diag_scan_kernel<bf16>, grid, dim3(1024), 0, stream, a, x, (const bf16*)yraw, ldy, ybias, state, state_stride,
                     (bf16*)out, seq_start, seq_slot, W));
}

// ------------------------------------------------------------------------------------------------ gated delta rule
// What the delta rule's recurrence takes, worked out per token in fp32 from the convolved projections:
//   qn = q / sqrt(sum q^2 + l2_eps) * q_scale and kn = k / sqrt(sum k^2 + l2_eps) per key head, qk = qn . kn,
//   dec[h, n] = -exp(A_log[h]) * softplus(z[h, n] + dt_bias[h, n]),  beta[h] = sigmoid(braw[h]).
// dec is the decay's logarithm: a float next to 1 has lost the digits of its distance from 1, which a state that lasts
// long depends on; the recurrence takes S + expm1(dec) S.  One block per token; a warp per key head, then per head.
template <typename T>
__global__ void __launch_bounds__(128)
delta_prep_kernel(const T* __restrict__ q, long ldq, const T* __restrict__ k, long ldk, const T* __restrict__ z, long ldz,
                  const T* __restrict__ braw, long ldb, const float* __restrict__ a_log, const float* __restrict__ dt_bias,
                  float l2_eps, float q_scale, float* __restrict__ qn, float* __restrict__ kn, float* __restrict__ qk,
                  float* __restrict__ dec, float* __restrict__ beta, int G, int H, int N) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int job = warp; job < G + H; job += 4) {
        if (job < G) {
            const T* qr = q + (long)t * ldq + (long)job * N;
            const T* kr = k + (long)t * ldk + (long)job * N;
            float sq = 0.f, sk = 0.f, sqk = 0.f;
            for (int i = lane; i < N; i += 32) {
                const float a = to_f32<T>(qr[i]), b = to_f32<T>(kr[i]);
                sq = fmaf(a, a, sq), sk = fmaf(b, b, sk), sqk = fmaf(a, b, sqk);
            }
            sq = warp_sum(sq), sk = warp_sum(sk), sqk = warp_sum(sqk);
            const float rq = q_scale / sqrtf(sq + l2_eps), rk = 1.0f / sqrtf(sk + l2_eps);
            float* qo = qn + ((long)t * G + job) * N;
            float* ko = kn + ((long)t * G + job) * N;
            for (int i = lane; i < N; i += 32) {
                qo[i] = to_f32<T>(qr[i]) * rq;
                ko[i] = to_f32<T>(kr[i]) * rk;
            }
            if (lane == 0) qk[(long)t * G + job] = sqk * rq * rk;
        } else {
            const int h = job - G;
            const float rate = expf(a_log[h]);
            const T* zr = z + (long)t * ldz + (long)h * N;
            float* d = dec + ((long)t * H + h) * N;
            for (int i = lane; i < N; i += 32) d[i] = -rate * softplus_f(to_f32<T>(zr[i]) + dt_bias[(long)h * N + i]);
            if (lane == 0) beta[(long)t * H + h] = sigmoid_f(to_f32<T>(braw[(long)t * ldb + h]));
        }
    }
}

extern "C" int plm_delta_prep(const void* q, long ldq, const void* k, long ldk, const void* z, long ldz, const void* braw, long ldb,
                              int dtype, const float* a_log, const float* dt_bias, float l2_eps, float q_scale, float* qn, float* kn,
                              float* qk, float* dec, float* beta, int n_tokens, int G, int H, int N, cudaStream_t stream) {
    if (n_tokens <= 0) return PLM_OK;
    if (G <= 0 || H <= 0 || N <= 0) return PLM_ERR_SHAPE;
    if (dtype == PLM_F32)
        return plm_status_of(launch_pdl(delta_prep_kernel<float>, dim3(n_tokens), dim3(128), 0, stream, (const float*)q, ldq,
                                        (const float*)k, ldk, (const float*)z, ldz, (const float*)braw, ldb, a_log, dt_bias, l2_eps,
                                        q_scale, qn, kn, qk, dec, beta, G, H, N));
    if (dtype == PLM_BF16)
        return plm_status_of(launch_pdl(delta_prep_kernel<bf16>, dim3(n_tokens), dim3(128), 0, stream, (const bf16*)q, ldq,
                                        (const bf16*)k, ldk, (const bf16*)z, ldz, (const bf16*)braw, ldb, a_log, dt_bias, l2_eps,
                                        q_scale, qn, kn, qk, dec, beta, G, H, N));
    return PLM_ERR_DTYPE;
}

// The delta rule per head, token by token, state S [N, P] in fp32:
//   S <- S + diag(expm1(dec_t)) S;  u = beta_t (v_t - S^T k_t);  S <- S + k_t u^T;  o_t = S^T q_t  (the read-out sees the
//   write; dec_t is the decay's logarithm).
// The columns of S do not meet, so a block takes 32 of them for one (sequence, head): a warp holds 8 columns, the N rows of
// a column are dealt to 4 lanes (row n with lane n % 4), NR values of the state a thread.  Both sums over the rows,
// k . (dec S) and q . (dec S), are taken in one pass before the write, and o = q . (dec S) + (q . k) u.
#define DELTA_COLS 32
template <typename T, int NR>
__global__ void __launch_bounds__(128)
delta_scan_kernel(const float* __restrict__ qn, const float* __restrict__ kn, const float* __restrict__ qk,
                  const float* __restrict__ dec, const float* __restrict__ beta, const T* __restrict__ v, long ldv,
                  float* __restrict__ state, long state_stride, float* __restrict__ y, const int* __restrict__ seq_start,
                  const int* __restrict__ seq_slot, int H, int N, int P, int heads_per_group, int TC) {
    constexpr int NP = NR * 4;
    extern __shared__ __align__(16) float smem[];
    float* qs = smem;                         // [TC][NP]
    float* ks = qs + (long)TC * NP;
    float* gs = ks + (long)TC * NP;
    float* vs = gs + (long)TC * NP;           // [TC][DELTA_COLS]
    float* bs = vs + (long)TC * DELTA_COLS;   // [TC] beta, then [TC] q . k
    pdl_launch_dependents();
    const int ptiles = (P + DELTA_COLS - 1) / DELTA_COLS;
    int bid = blockIdx.x;
    const int ptile = bid % ptiles;
    bid /= ptiles;
    const int h = bid % H, b = bid / H;
    const int g = h / heads_per_group, G = H / heads_per_group;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int col = (warp << 3) + (lane & 7), part = lane >> 3;
    const int p = ptile * DELTA_COLS + col;
    pdl_wait();
    const int s0 = seq_start[b], s1 = seq_start[b + 1];
    if (s1 <= s0) return;
    float* st = state + (long)seq_slot[b] * state_stride + (long)h * N * P;
    float S[NR];
#pragma unroll
    for (int r = 0; r < NR; ++r) {
        const int n = r * 4 + part;
        S[r] = (n < N && p < P) ? st[(long)n * P + p] : 0.f;
    }
    for (int base = s0; base < s1; base += TC) {
        const int nt = min(TC, s1 - base);
        __syncthreads();
        for (int idx = threadIdx.x; idx < nt * NP; idx += 128) {
            const int tt = idx / NP, n = idx - tt * NP;
            const long row = base + tt;
            const bool in = n < N;
            qs[idx] = in ? qn[(row * G + g) * N + n] : 0.f;
            ks[idx] = in ? kn[(row * G + g) * N + n] : 0.f;
            gs[idx] = in ? expm1f(dec[(row * H + h) * N + n]) : 0.f;
        }
        for (int idx = threadIdx.x; idx < nt * DELTA_COLS; idx += 128) {
            const int tt = idx / DELTA_COLS, cc = idx - tt * DELTA_COLS;
            const int pp = ptile * DELTA_COLS + cc;
            vs[idx] = pp < P ? to_f32<T>(v[(long)(base + tt) * ldv + (long)h * P + pp]) : 0.f;
        }
        for (int tt = threadIdx.x; tt < nt; tt += 128) {
            bs[tt] = beta[(long)(base + tt) * H + h];
            bs[TC + tt] = qk[(long)(base + tt) * G + g];
        }
        __syncthreads();
        for (int tt = 0; tt < nt; ++tt) {
            const float* qt = qs + tt * NP + part;
            const float* kt = ks + tt * NP + part;
            const float* gt = gs + tt * NP + part;
            float d1 = 0.f, d2 = 0.f;
#pragma unroll
            for (int r = 0; r < NR; ++r) {
                const float s = fmaf(S[r], gt[r * 4], S[r]);
                S[r] = s;
                d1 = fmaf(kt[r * 4], s, d1);
                d2 = fmaf(qt[r * 4], s, d2);
            }
            d1 += __shfl_xor_sync(0xffffffffu, d1, 8);
            d2 += __shfl_xor_sync(0xffffffffu, d2, 8);
            d1 += __shfl_xor_sync(0xffffffffu, d1, 16);
            d2 += __shfl_xor_sync(0xffffffffu, d2, 16);
            const float u = bs[tt] * (vs[tt * DELTA_COLS + col] - d1);
#pragma unroll
            for (int r = 0; r < NR; ++r) S[r] = fmaf(kt[r * 4], u, S[r]);
            if (part == 0 && p < P) y[(long)(base + tt) * H * P + (long)h * P + p] = fmaf(bs[TC + tt], u, d2);
        }
    }
#pragma unroll
    for (int r = 0; r < NR; ++r) {
        const int n = r * 4 + part;
        if (n < N && p < P) st[(long)n * P + p] = S[r];
    }
}

template <typename T, int NR>
static int delta_scan_launch(const float* qn, const float* kn, const float* qk, const float* dec, const float* beta, const void* v,
                             long ldv, float* state, long state_stride, float* y, const int* seq_start, const int* seq_slot,
                             int n_seqs, int H, int N, int P, int heads_per_group, cudaStream_t stream) {
    const int TC = NR <= 32 ? 16 : 8;
    const size_t smem = ((size_t)TC * NR * 4 * 3 + (size_t)TC * DELTA_COLS + 2 * TC) * sizeof(float);
    if (smem > 48 * 1024)
        cudaFuncSetAttribute(delta_scan_kernel<T, NR>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    const unsigned grid = (unsigned)((long)n_seqs * H * ((P + DELTA_COLS - 1) / DELTA_COLS));
    return plm_status_of(launch_pdl(delta_scan_kernel<T, NR>, dim3(grid), dim3(128), smem, stream, qn, kn, qk, dec, beta,
                                    (const T*)v, ldv, state, state_stride, y, seq_start, seq_slot, H, N, P, heads_per_group, TC));
}

extern "C" int plm_delta_scan(const float* qn, const float* kn, const float* qk, const float* dec, const float* beta,
                              const void* v, int dtype, long ldv, float* state, long state_stride, float* y, const int* seq_start,
                              const int* seq_slot, int n_seqs, int H, int N, int P, int heads_per_group, cudaStream_t stream) {
    if (n_seqs <= 0) return PLM_OK;
    if (H <= 0 || N <= 0 || P <= 0 || heads_per_group <= 0 || H % heads_per_group) return PLM_ERR_SHAPE;
    if (N > 256) return PLM_ERR_UNSUPPORTED;
    if (dtype != PLM_F32 && dtype != PLM_BF16) return PLM_ERR_DTYPE;
    const int nr = (N + 3) / 4;
#define DS(NR_)                                                                                                                 \
    return dtype == PLM_F32                                                                                                     \
               ? delta_scan_launch<float, NR_>(qn, kn, qk, dec, beta, v, ldv, state, state_stride, y, seq_start, seq_slot, n_seqs, \
                                               H, N, P, heads_per_group, stream)                                               \
               : delta_scan_launch<bf16, NR_>(qn, kn, qk, dec, beta, v, ldv, state, state_stride, y, seq_start, seq_slot, n_seqs, \
                                              H, N, P, heads_per_group, stream)
    if (nr <= 4) DS(4);
    if (nr <= 8) DS(8);
    if (nr <= 16) DS(16);
    if (nr <= 24) DS(24);
    if (nr <= 32) DS(32);
    if (nr <= 48) DS(48);
    DS(64);
#undef DS
}

// ------------------------------------------------------------------------------------- gated delta rule, chunk by chunk
// The same recurrence for prompts, DELTA_CHUNK tokens at a time.  With L_t the running sum of the decays' logarithms
// inside a chunk (per head and key channel) and S_0 the state the chunk starts from,
//   u_t = beta_t (v_t - S_0^T (k_t e^{L_t}) - sum_{s<t} A_ts u_s),   A_ts = sum_n k_tn k_sn e^{L_tn - L_sn}
//   o_t = S_0^T (q_t e^{L_t}) + sum_{s<=t} M_ts u_s,                 M_ts = sum_n q_tn k_sn e^{L_tn - L_sn}
//   S_C = diag(e^{L_C}) S_0 + sum_s (k_s e^{L_C - L_s}) u_s^T
// Every exponent is <= 0: nothing is divided by a running decay, so no choice of decays overflows.  What does not depend
// on the state (the three scaled copies of k and q, A, M, e^{L_C}) is made for all chunks side by side by a first
// kernel; the second walks a sequence's chunks with the state in registers: two passes of dot products without a chain
// between tokens, a forward substitution over the chunk's tokens, and the state's update.
#define DELTA_CHUNK 32

__host__ __device__ static inline long delta_ws_floats(int NP) { return 3L * DELTA_CHUNK * NP + 2L * DELTA_CHUNK * DELTA_CHUNK + NP; }

// The width of a row of keys in the workspace: eight times the NR values a thread of the second kernel holds.
static inline int delta_chunk_np(int N) { return N <= 32 ? 32 : N <= 64 ? 64 : N <= 128 ? 128 : 256; }

// grid (chunk of the sequence, sequence, head).  ws per (slot, head): Kp [C][NP] | Qp [C][NP] | Ke [C][NP] | A^T [C][C] | M^T [C][C]
// | e^{L_C} [NP], NP = delta_chunk_np(N), the padding zero.  A sequence's chunk c lives in slot seq_start / C + sequence + c.
__global__ void __launch_bounds__(256)
delta_chunk_prep_kernel(const float* __restrict__ qn, const float* __restrict__ kn, const float* __restrict__ lgd,
                        float* __restrict__ ws, const int* __restrict__ seq_start, int H, int N, int NP, int heads_per_group) {
    constexpr int C = DELTA_CHUNK;
    extern __shared__ __align__(16) float smem[];
    float* cum = smem;                  // [C][N]
    float* ks = cum + (long)C * N;
    float* qs = ks + (long)C * N;
    pdl_launch_dependents();
    pdl_wait();
    const int c = blockIdx.x, b = blockIdx.y, h = blockIdx.z;
    const int s0 = seq_start[b], s1 = seq_start[b + 1];
    const int t0 = s0 + c * C;
    if (t0 >= s1) return;
    const int nt = min(C, s1 - t0);
    const int G = H / heads_per_group, g = h / heads_per_group;
    const long slot = (long)(s0 / C) + b + c;
    for (int idx = threadIdx.x; idx < C * N; idx += 256) {
        const int tt = idx / N, n = idx - tt * N;
        const bool in = tt < nt;
        const long row = t0 + tt;
        ks[idx] = in ? kn[(row * G + g) * N + n] : 0.f;
        qs[idx] = in ? qn[(row * G + g) * N + n] : 0.f;
        cum[idx] = in ? lgd[(row * H + h) * N + n] : 0.f;
    }
    __syncthreads();
    for (int n = threadIdx.x; n < N; n += 256) {
        float acc = 0.f;
        for (int tt = 0; tt < C; ++tt) {
            acc += cum[tt * N + n];
            cum[tt * N + n] = acc;
        }
    }
    __syncthreads();
    float* out = ws + (slot * H + h) * delta_ws_floats(NP);
    float* Kp = out;
    float* Qp = Kp + (long)C * NP;
    float* Ke = Qp + (long)C * NP;
    float* A = Ke + (long)C * NP;
    float* M = A + C * C;
    float* ge = M + C * C;
    for (int idx = threadIdx.x; idx < C * NP; idx += 256) {
        const int tt = idx / NP, n = idx - tt * NP;
        float kp = 0.f, qp = 0.f, ke = 0.f;
        if (n < N) {
            const float l = cum[tt * N + n], e = expf(l), kv = ks[tt * N + n];
            kp = kv * e;
            qp = qs[tt * N + n] * e;
            ke = kv * expf(cum[(C - 1) * N + n] - l);
        }
        Kp[idx] = kp, Qp[idx] = qp, Ke[idx] = ke;
    }
    for (int n = threadIdx.x; n < NP; n += 256) ge[n] = n < N ? expf(cum[(C - 1) * N + n]) : 0.f;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // both stored transposed, [s][t], so that lanes that hold different t read different banks; zero where s > t (A: s >= t)
    for (int i = warp; i < C * C; i += 8) {
        const int t = i / C, s = i - t * C;
        float a = 0.f, m = 0.f;
        if (s <= t) {
            for (int n = lane; n < N; n += 32) {
                const float kk = ks[s * N + n] * expf(cum[t * N + n] - cum[s * N + n]);
                a = fmaf(ks[t * N + n], kk, a);
                m = fmaf(qs[t * N + n], kk, m);
            }
            a = warp_sum(a), m = warp_sum(m);
        }
        if (lane == 0) A[s * C + t] = s < t ? a : 0.f, M[s * C + t] = m;
    }
}

// grid: (sequence, head, DELTA_CCOLS columns of the state).  A warp holds 4 columns; the N rows of a column are dealt to 8
// lanes in contiguous eighths, NR values of the state a thread.  A chunk's matrices come through cp.async into one of
// STAGES buffers, the next chunk's while this one is worked on.
#define DELTA_CCOLS 16
__device__ __forceinline__ void cp_async16(float* dst, const float* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}

template <int NR, int STAGES>
__global__ void __launch_bounds__(128)
delta_chunk_scan_kernel(const float* __restrict__ ws, const float* __restrict__ beta, const void* __restrict__ v, int v_f32, long ldv,
                        float* __restrict__ state, long state_stride, float* __restrict__ y, const int* __restrict__ seq_start,
                        const int* __restrict__ seq_slot, int H, int N, int P) {
    constexpr int C = DELTA_CHUNK, NP = NR * 8, SEG = NR + 4, RS = 8 * SEG;      // SEG: an eighth's floats in a row, padded
    constexpr int STAGE = 3 * C * RS + 2 * C * C + RS;                            // Kp | Qp | Ke [C][RS], A | M [C][C], e^{L_C} [RS]
    extern __shared__ __align__(16) float smem[];
    float* vs = smem + STAGES * STAGE;   // [C][DELTA_CCOLS]
    float* bs = vs + C * DELTA_CCOLS;    // [C]
    pdl_launch_dependents();
    const int ptiles = (P + DELTA_CCOLS - 1) / DELTA_CCOLS;
    int bid = blockIdx.x;
    const int ptile = bid % ptiles;
    bid /= ptiles;
    const int h = bid % H, b = bid / H;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int col = (warp << 2) + (lane & 3), part = lane >> 2;
    const int p = ptile * DELTA_CCOLS + col;
    pdl_wait();
    const int s0 = seq_start[b], s1 = seq_start[b + 1];
    if (s1 <= s0) return;
    float* st = state + (long)seq_slot[b] * state_stride + (long)h * N * P;
    float S[NR];
#pragma unroll
    for (int j = 0; j < NR; ++j) {
        const int n = part * NR + j;
        S[j] = (n < N && p < P) ? st[(long)n * P + p] : 0.f;
    }
    const long wsf = 3L * C * NP + 2L * C * C + NP;
    const float* src0 = ws + (((long)(s0 / C) + b) * H + h) * wsf;
    const int n_chunks = (s1 - s0 + C - 1) / C;
    auto fetch = [&](int chunk, int stage) {
        const float* src = src0 + (long)chunk * H * wsf;
        float* dst = smem + stage * STAGE;
        constexpr int ROW4 = NP / 4, MAT4 = C * ROW4;
        for (int idx = threadIdx.x; idx < 3 * MAT4; idx += 128) {
            const int m = idx / MAT4, rem = idx - m * MAT4;
            const int tt = rem / ROW4, n4 = (rem - tt * ROW4) * 4;
            const int prt = n4 / NR, j = n4 - prt * NR;
            cp_async16(dst + m * C * RS + tt * RS + prt * SEG + j, src + (long)m * C * NP + (long)tt * NP + n4);
        }
        for (int idx = threadIdx.x; idx < 2 * C * C / 4; idx += 128) cp_async16(dst + 3 * C * RS + idx * 4, src + 3L * C * NP + idx * 4);
        for (int idx = threadIdx.x; idx < ROW4; idx += 128) {
            const int n4 = idx * 4, prt = n4 / NR, j = n4 - prt * NR;
            cp_async16(dst + 3 * C * RS + 2 * C * C + prt * SEG + j, src + 3L * C * NP + 2L * C * C + n4);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    if (STAGES == 2) fetch(0, 0);
    for (int chunk = 0; chunk < n_chunks; ++chunk) {
        const int base = s0 + chunk * C, nt = min(C, s1 - base);
        const int stage = STAGES == 2 ? (chunk & 1) : 0;
        if (STAGES == 2) {
            if (chunk + 1 < n_chunks) {
                fetch(chunk + 1, stage ^ 1);
                asm volatile("cp.async.wait_group 1;" ::: "memory");
            } else {
                asm volatile("cp.async.wait_group 0;" ::: "memory");
            }
        } else {
            fetch(chunk, 0);
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        for (int idx = threadIdx.x; idx < C * DELTA_CCOLS; idx += 128) {
            const int tt = idx / DELTA_CCOLS, cc = idx - tt * DELTA_CCOLS;
            const int pp = ptile * DELTA_CCOLS + cc;
            const long at = (long)(base + tt) * ldv + (long)h * P + pp;
            vs[idx] = (tt < nt && pp < P) ? (v_f32 ? static_cast<const float*>(v)[at] : to_f32<bf16>(static_cast<const bf16*>(v)[at])) : 0.f;
        }
        if (threadIdx.x < C) bs[threadIdx.x] = threadIdx.x < nt ? beta[(long)(base + threadIdx.x) * H + h] : 0.f;
        __syncthreads();
        const float* Kp = smem + stage * STAGE;
        const float* Qp = Kp + C * RS;
        const float* Ke = Qp + C * RS;
        const float* A = Ke + C * RS;
        const float* M = A + C * C;
        const float* ge = M + C * C;
        // this lane's share of both dot products for every token of the chunk
        float r[C], o[C];
#pragma unroll
        for (int t = 0; t < C; ++t) {
            const float4* kp = reinterpret_cast<const float4*>(Kp + t * RS + part * SEG);
            const float4* qp = reinterpret_cast<const float4*>(Qp + t * RS + part * SEG);
            float ra0 = 0.f, ra1 = 0.f, oa0 = 0.f, oa1 = 0.f;
#pragma unroll
            for (int j4 = 0; j4 < NR / 4; ++j4) {
                const float4 a = kp[j4], q = qp[j4];
                ra0 = fmaf(a.x, S[4 * j4], ra0), ra1 = fmaf(a.y, S[4 * j4 + 1], ra1);
                ra0 = fmaf(a.z, S[4 * j4 + 2], ra0), ra1 = fmaf(a.w, S[4 * j4 + 3], ra1);
                oa0 = fmaf(q.x, S[4 * j4], oa0), oa1 = fmaf(q.y, S[4 * j4 + 1], oa1);
                oa0 = fmaf(q.z, S[4 * j4 + 2], oa0), oa1 = fmaf(q.w, S[4 * j4 + 3], oa1);
            }
            r[t] = ra0 + ra1;
            o[t] = oa0 + oa1;
        }
        // The eight lanes of a column add their shares so that lane `part` ends with the sums of tokens 4 part .. 4 part + 3
        // (three rounds, each handing half of what is left to the partner): r[0..3], o[0..3].
#pragma unroll
        for (int half = C / 2, mask = 16; half >= 4; half >>= 1, mask >>= 1) {
            const bool upper = (lane & mask) != 0;
#pragma unroll
            for (int i = 0; i < half; ++i) {
                const float sr = upper ? r[i] : r[i + half], so = upper ? o[i] : o[i + half];
                const float kr = upper ? r[i + half] : r[i], ko = upper ? o[i + half] : o[i];
                r[i] = kr + __shfl_xor_sync(0xffffffffu, sr, mask);
                o[i] = ko + __shfl_xor_sync(0xffffffffu, so, mask);
            }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) r[j] = vs[(part * 4 + j) * DELTA_CCOLS + col] - r[j];
        // forward substitution: the owner of token t makes u_t and hands it to the column's other lanes; every lane
        // keeps all of u and takes u_t out of the tokens it owns (A^T is zero where they are not later than t)
        float u[C];
#pragma unroll
        for (int t = 0; t < C; ++t) {
            u[t] = __shfl_sync(0xffffffffu, bs[t] * r[t & 3], ((t >> 2) << 2) + (lane & 3));
            const float* at = A + t * C + part * 4;
#pragma unroll
            for (int j = 0; j < 4; ++j) r[j] = fmaf(-at[j], u[t], r[j]);
        }
        {
            float acc[4] = {o[0], o[1], o[2], o[3]};
#pragma unroll
            for (int s = 0; s < C; ++s) {
                const float* mt = M + s * C + part * 4;
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[j] = fmaf(mt[j], u[s], acc[j]);
            }
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (p < P && part * 4 + j < nt) y[(long)(base + part * 4 + j) * H * P + (long)h * P + p] = acc[j];
        }
#pragma unroll
        for (int j = 0; j < NR; ++j) S[j] *= ge[part * SEG + j];
#pragma unroll
        for (int s = 0; s < C; ++s) {
            const float4* ke = reinterpret_cast<const float4*>(Ke + s * RS + part * SEG);
#pragma unroll
            for (int j4 = 0; j4 < NR / 4; ++j4) {
                const float4 e = ke[j4];
                S[4 * j4] = fmaf(e.x, u[s], S[4 * j4]), S[4 * j4 + 1] = fmaf(e.y, u[s], S[4 * j4 + 1]);
                S[4 * j4 + 2] = fmaf(e.z, u[s], S[4 * j4 + 2]), S[4 * j4 + 3] = fmaf(e.w, u[s], S[4 * j4 + 3]);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int j = 0; j < NR; ++j) {
        const int n = part * NR + j;
        if (n < N && p < P) st[(long)n * P + p] = S[j];
    }
}

template <int NR, int STAGES>
static int delta_chunk_launch(const float* ws, const float* beta, const void* v, int v_f32, long ldv, float* state, long state_stride,
                              float* y, const int* seq_start, const int* seq_slot, int n_seqs, int H, int N, int P,
                              cudaStream_t stream) {
    constexpr int C = DELTA_CHUNK, RS = 8 * (NR + 4);
    const size_t smem = ((size_t)STAGES * (3 * C * RS + 2 * C * C + RS) + C * DELTA_CCOLS + C) * sizeof(float);
    if (smem > 48 * 1024)
        cudaFuncSetAttribute(delta_chunk_scan_kernel<NR, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    const unsigned grid = (unsigned)((long)n_seqs * H * ((P + DELTA_CCOLS - 1) / DELTA_CCOLS));
    return plm_status_of(launch_pdl(delta_chunk_scan_kernel<NR, STAGES>, dim3(grid), dim3(128), smem, stream, ws, beta, v, v_f32,
                                    ldv, state, state_stride, y, seq_start, seq_slot, H, N, P));
}

// ws: ((n_tokens / DELTA_CHUNK) + n_seqs + 1) * H * delta_ws_floats(delta_chunk_np(N)) floats.
extern "C" int plm_delta_chunk_scan(const float* qn, const float* kn, const float* dec, const float* beta, const void* v,
                                    int dtype, long ldv, float* state, long state_stride, float* y, float* ws,
                                    const int* seq_start, const int* seq_slot, int n_seqs, int max_new, int H, int N, int P,
                                    int heads_per_group, cudaStream_t stream) {
    if (n_seqs <= 0 || max_new <= 0) return PLM_OK;
    if (H <= 0 || N <= 0 || P <= 0 || heads_per_group <= 0 || H % heads_per_group) return PLM_ERR_SHAPE;
    if (N > 256) return PLM_ERR_UNSUPPORTED;
    if (dtype != PLM_F32 && dtype != PLM_BF16) return PLM_ERR_DTYPE;
    const int NP = delta_chunk_np(N);
    const size_t prep_smem = (size_t)3 * DELTA_CHUNK * N * sizeof(float);
    if (prep_smem > 48 * 1024)
        cudaFuncSetAttribute(delta_chunk_prep_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)prep_smem);
    const dim3 pgrid((unsigned)((max_new + DELTA_CHUNK - 1) / DELTA_CHUNK), (unsigned)n_seqs, (unsigned)H);
    int e = plm_status_of(launch_pdl(delta_chunk_prep_kernel, pgrid, dim3(256), prep_smem, stream, qn, kn, dec, ws, seq_start, H, N,
                                     NP, heads_per_group));
    if (e != PLM_OK) return e;
#define DCS(NR_, ST_)                                                                                                     \
    return delta_chunk_launch<NR_, ST_>(ws, beta, v, dtype == PLM_F32 ? 1 : 0, ldv, state, state_stride, y, seq_start, seq_slot, \
                                        n_seqs, H, N, P, stream)
    if (NP <= 32) DCS(4, 2);
    if (NP <= 64) DCS(8, 2);
    if (NP <= 128) DCS(16, 2);
    DCS(32, 1);
#undef DCS
}
