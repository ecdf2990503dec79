// Row-wise and element-wise kernels of the decoder: token embedding gather,
// RMSNorm with the residual add folded in, SwiGLU, and rotary position
// encoding fused with the write of K and V into the paged cache.
//
// Formulas follow the reference's scalar forms:
//   RMSNorm   ss = sum x^2; r = 1/sqrtf(ss/size + eps); out = (x*r)*w   (picolm/tensor.c:2942-3064)
//   SiLU      x / (1 + expf(-x)), multiplied by the up branch             (picolm/tensor.c:3306-3315,
//                                                                          picolm/model_core.c:2192-2193)
//   RoPE      (x0,x1) -> (x0*c - x1*s, x0*s + x1*c), q and k only         (picolm/tensor.c:3216-3304)
//   embedding x = float(row of the table), no scale                       (picolm/model_core.c:1785-1786)
// All statistics and the residual stream are fp32.
#include "common.cuh"

// ------------------------------------------------------------------ embedding
template <typename Tw>
__global__ void embed_kernel(const int* __restrict__ tok, const Tw* __restrict__ table, float* __restrict__ out,
                             int d, int vocab, float scale) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    int id = tok[t];
    if (id < 0 || id >= vocab) id = 0;   // ids are checked on the host; never read outside the table
    const Tw* row = table + (size_t)id * d;
    float* o = out + (size_t)t * d;
    // (a scale of 1 changes nothing: the product with 1.0f is exact)
    for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = __fmul_rn(to_f32<Tw>(row[i]), scale);
}

// out[t, :] = float(table[tok[t], :]) * scale (the reference has no scale; a design that multiplies its embeddings
// by a constant gives it here)
extern "C" int plm_embed(const int* tok, const void* table, int table_dtype, float* out, int n_tokens, int d,
                         int vocab, float scale, cudaStream_t stream) {
    if (n_tokens <= 0) return PLM_OK;
    if (d <= 0 || vocab <= 0) return PLM_ERR_SHAPE;
    const int nt = d >= 1024 ? 256 : 128;
    if (table_dtype == PLM_F32)
        return plm_status_of(launch_pdl(embed_kernel<float>, n_tokens, nt, 0, stream, tok, (const float*)table, out, d, vocab, scale));
    if (table_dtype == PLM_BF16)
        return plm_status_of(launch_pdl(embed_kernel<bf16>, n_tokens, nt, 0, stream, tok, (const bf16*)table, out, d, vocab, scale));
    return PLM_ERR_DTYPE;
}

// -------------------------------------------------------------------- RMSNorm
// One block per output row.  Row r reads source row rows[r] (or r).  With a
// delta the sum x + delta is normalised; it is written back to x unless rows are
// gathered.  The reduction order depends on the row's width only, never on what
// else is in the batch.

template <typename Tw, typename To, int NT>
__global__ void rmsnorm_kernel(float* __restrict__ x, const float* __restrict__ delta, const Tw* __restrict__ w,
                               To* __restrict__ out, const int* __restrict__ rows, int d, float eps, int write_back) {
    __shared__ float red[33];
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    const int src = rows ? PLM_ROW_NO(rows[r]) : r;
    float* xr = x + (size_t)src * d;
    const float* dr = delta ? delta + (size_t)src * d : nullptr;
    float ss = 0.f;
    for (int i = threadIdx.x; i < d; i += NT) {
        float v = xr[i];
        if (dr) {
            v += dr[i];
            if (write_back) xr[i] = v;
        }
        ss += v * v;
    }
    ss = block_sum<NT>(ss, red);
    const float scale = 1.0f / sqrtf(ss / (float)d + eps);
    To* o = out + (size_t)r * d;
    for (int i = threadIdx.x; i < d; i += NT) {
        float v = xr[i];
        if (dr && !write_back) v += dr[i];
        o[i] = from_f32<To>(v * scale * to_f32<Tw>(w[i]));
    }
}

// Four elements at a time, the row kept in registers between the two passes: for rows whose width
// is a multiple of 4 and at most 16 * NT.
__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const bf16* p) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&u.x), b = *reinterpret_cast<const __nv_bfloat162*>(&u.y);
    return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(bf16* p, float4 v) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 u;
    u.x = *reinterpret_cast<uint32_t*>(&a);
    u.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = u;
}

template <typename Tw, typename To, int NT>
__global__ void __launch_bounds__(NT)
rmsnorm_vec_kernel(float* __restrict__ x, const float* __restrict__ delta, const Tw* __restrict__ w,
                   To* __restrict__ out, const int* __restrict__ rows, int d, float eps, int write_back) {
    __shared__ float red[33];
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    const int src = rows ? PLM_ROW_NO(rows[r]) : r;
    float* xr = x + (size_t)src * d;
    const float* dr = delta ? delta + (size_t)src * d : nullptr;
    float4 v[4];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int i = (threadIdx.x + k * NT) * 4;
        if (i < d) {
            v[k] = load4(xr + i);
            if (dr) {
                const float4 dv = load4(dr + i);
                v[k].x += dv.x; v[k].y += dv.y; v[k].z += dv.z; v[k].w += dv.w;
                if (write_back) store4(xr + i, v[k]);
            }
            ss += v[k].x * v[k].x + v[k].y * v[k].y + v[k].z * v[k].z + v[k].w * v[k].w;
        }
    }
    ss = block_sum<NT>(ss, red);
    const float scale = 1.0f / sqrtf(ss / (float)d + eps);
    To* o = out + (size_t)r * d;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int i = (threadIdx.x + k * NT) * 4;
        if (i < d) {
            const float4 wv = load4(w + i);
            store4(o + i, make_float4(v[k].x * scale * wv.x, v[k].y * scale * wv.y, v[k].z * scale * wv.z,
                                      v[k].w * scale * wv.w));
        }
    }
}

template <typename Tw, typename To>
static int rmsnorm_launch(float* x, const float* delta, const void* w, void* out, const int* rows, int n_rows, int d,
                          float eps, int write_back, cudaStream_t stream) {
    if (d % 4 == 0 && d <= 16 * 1024) {
        // the block size (and with it the order of the sum of squares) depends on the row's width only
        if (d <= 16 * 256)
            return plm_status_of(launch_pdl(rmsnorm_vec_kernel<Tw, To, 256>, n_rows, 256, 0, stream, x, delta,
                                            (const Tw*)w, (To*)out, rows, d, eps, write_back));
        return plm_status_of(launch_pdl(rmsnorm_vec_kernel<Tw, To, 1024>, n_rows, 1024, 0, stream, x, delta,
                                        (const Tw*)w, (To*)out, rows, d, eps, write_back));
    }
    // enough threads that a row's loads are all in flight at once; the block size (and with it the
    // order of the sum of squares) depends on the row's width only
    if (d > 1024)
        return plm_status_of(launch_pdl(rmsnorm_kernel<Tw, To, 1024>, n_rows, 1024, 0, stream, x, delta,
                                        (const Tw*)w, (To*)out, rows, d, eps, write_back));
    return plm_status_of(launch_pdl(rmsnorm_kernel<Tw, To, 256>, n_rows, 256, 0, stream, x, delta, (const Tw*)w,
                                    (To*)out, rows, d, eps, write_back));
}

extern "C" int plm_rmsnorm(float* x, const float* delta, const void* w, int w_dtype, void* out, int out_dtype,
                           const int* rows, int n_rows, int d, float eps, cudaStream_t stream) {
    if (n_rows <= 0) return PLM_OK;
    if (d <= 0) return PLM_ERR_SHAPE;
    const int write_back = (delta != nullptr && rows == nullptr) ? 1 : 0;
    if (w_dtype == PLM_F32 && out_dtype == PLM_F32)
        return rmsnorm_launch<float, float>(x, delta, w, out, rows, n_rows, d, eps, write_back, stream);
    if (w_dtype == PLM_BF16 && out_dtype == PLM_F32)
        return rmsnorm_launch<bf16, float>(x, delta, w, out, rows, n_rows, d, eps, write_back, stream);
    if (w_dtype == PLM_F32 && out_dtype == PLM_BF16)
        return rmsnorm_launch<float, bf16>(x, delta, w, out, rows, n_rows, d, eps, write_back, stream);
    if (w_dtype == PLM_BF16 && out_dtype == PLM_BF16)
        return rmsnorm_launch<bf16, bf16>(x, delta, w, out, rows, n_rows, d, eps, write_back, stream);
    return PLM_ERR_DTYPE;
}

// A sublayer's result normalised, added to the stream, and the new stream normalised for the next sublayer, in
// one pass over the row: x += (delta * r1) * w_post with r1 from delta's mean square; out = (x * r2) * w_pre with
// r2 from the new x's.  The same roundings as the two kernels it replaces (each product rounded, then the sum).
// Rows whose width is a multiple of 4 and at most 16 * NT stay in registers throughout.
template <typename Tw, typename To, int NT>
__global__ void __launch_bounds__(NT)
post_pre_norm_kernel(float* __restrict__ x, const float* __restrict__ delta, const Tw* __restrict__ w_post,
                     const Tw* __restrict__ w_pre, To* __restrict__ out, int d, float eps_post, float eps_pre) {
    __shared__ float red[33];
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    float* xr = x + (size_t)r * d;
    const float* dr = delta + (size_t)r * d;
    float4 v[4];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int i = (threadIdx.x + k * NT) * 4;
        if (i < d) {
            v[k] = load4(dr + i);
            ss += v[k].x * v[k].x + v[k].y * v[k].y + v[k].z * v[k].z + v[k].w * v[k].w;
        }
    }
    ss = block_sum<NT>(ss, red);
    const float s1 = 1.0f / sqrtf(ss / (float)d + eps_post);
    ss = 0.f;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int i = (threadIdx.x + k * NT) * 4;
        if (i < d) {
            const float4 wv = load4(w_post + i), xv = load4(xr + i);
            v[k].x = __fadd_rn(xv.x, __fmul_rn(__fmul_rn(v[k].x, s1), wv.x));
            v[k].y = __fadd_rn(xv.y, __fmul_rn(__fmul_rn(v[k].y, s1), wv.y));
            v[k].z = __fadd_rn(xv.z, __fmul_rn(__fmul_rn(v[k].z, s1), wv.z));
            v[k].w = __fadd_rn(xv.w, __fmul_rn(__fmul_rn(v[k].w, s1), wv.w));
            store4(xr + i, v[k]);
            ss += v[k].x * v[k].x + v[k].y * v[k].y + v[k].z * v[k].z + v[k].w * v[k].w;
        }
    }
    ss = block_sum<NT>(ss, red);
    const float s2 = 1.0f / sqrtf(ss / (float)d + eps_pre);
    To* o = out + (size_t)r * d;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int i = (threadIdx.x + k * NT) * 4;
        if (i < d) {
            const float4 wv = load4(w_pre + i);
            store4(o + i, make_float4(v[k].x * s2 * wv.x, v[k].y * s2 * wv.y, v[k].z * s2 * wv.z, v[k].w * s2 * wv.w));
        }
    }
}

template <typename Tw, typename To>
static int post_pre_norm_launch(float* x, const float* delta, const void* w_post, const void* w_pre, void* out, int n_rows,
                                int d, float eps_post, float eps_pre, cudaStream_t stream) {
    if (d <= 16 * 256)
        return plm_status_of(launch_pdl(post_pre_norm_kernel<Tw, To, 256>, n_rows, 256, 0, stream, x, delta, (const Tw*)w_post,
                                        (const Tw*)w_pre, (To*)out, d, eps_post, eps_pre));
    return plm_status_of(launch_pdl(post_pre_norm_kernel<Tw, To, 1024>, n_rows, 1024, 0, stream, x, delta, (const Tw*)w_post,
                                    (const Tw*)w_pre, (To*)out, d, eps_post, eps_pre));
}

extern "C" int plm_post_pre_norm(float* x, const float* delta, const void* w_post, const void* w_pre, int w_dtype, void* out,
                                 int out_dtype, int n_rows, int d, float eps_post, float eps_pre, cudaStream_t stream) {
    if (n_rows <= 0) return PLM_OK;
    if (d <= 0 || d % 4 || d > 16 * 1024) return PLM_ERR_SHAPE;
    if (w_dtype == PLM_F32 && out_dtype == PLM_F32)
        return post_pre_norm_launch<float, float>(x, delta, w_post, w_pre, out, n_rows, d, eps_post, eps_pre, stream);
    if (w_dtype == PLM_BF16 && out_dtype == PLM_F32)
        return post_pre_norm_launch<bf16, float>(x, delta, w_post, w_pre, out, n_rows, d, eps_post, eps_pre, stream);
    if (w_dtype == PLM_F32 && out_dtype == PLM_BF16)
        return post_pre_norm_launch<float, bf16>(x, delta, w_post, w_pre, out, n_rows, d, eps_post, eps_pre, stream);
    if (w_dtype == PLM_BF16 && out_dtype == PLM_BF16)
        return post_pre_norm_launch<bf16, bf16>(x, delta, w_post, w_pre, out, n_rows, d, eps_post, eps_pre, stream);
    return PLM_ERR_DTYPE;
}

// ------------------------------------------------ rows whose scale is still due
// out[t, :] = bf16(x[t, :] * r[t]) with r[t] = 1 / sqrt(sum_p parts[p, t] / size + eps): what is left of
// an RMSNorm whose weight a product's epilogue has already applied (x) and whose sums of squares it has
// left as partial sums (parts [n_parts, ld_parts]).  One block per row, sums in a fixed order.
__global__ void scale_rows_kernel(const bf16* __restrict__ x, const float* __restrict__ parts, int n_parts, int ld_parts,
                                  float inv_size, float eps, bf16* __restrict__ out, int d) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    float ss = 0.f;
    for (int p = 0; p < n_parts; ++p) ss += parts[(size_t)p * ld_parts + t];
    const float r = 1.0f / sqrtf(ss * inv_size + eps);
    for (int i = threadIdx.x; i < d; i += blockDim.x)
        out[(size_t)t * d + i] = __float2bfloat16_rn(__bfloat162float(x[(size_t)t * d + i]) * r);
}

extern "C" int plm_scale_rows(const void* x, const float* parts, int n_parts, int ld_parts, int size, float eps,
                              void* out, int n_rows, int d, cudaStream_t stream) {
    if (n_rows <= 0) return PLM_OK;
    if (d <= 0 || size <= 0 || n_parts <= 0 || ld_parts < n_rows) return PLM_ERR_SHAPE;
    return plm_status_of(launch_pdl(scale_rows_kernel, dim3(n_rows), dim3(256), 0, stream, (const bf16*)x, parts, n_parts,
                                    ld_parts, 1.0f / (float)size, eps, (bf16*)out, d));
}

// ----------------------------------------------------------- gated activation
// gu is [T, 2F]: gate in columns [0,F), up in [F,2F).  out[T,F] = act(gate) * up, with
// ACT 0: silu(g) = g / (1 + expf(-g))                                  (picolm/tensor.c:3306-3315)
// ACT 1: gelu(g) = 0.5 g (1 + tanhf(0.79788456 (g + 0.044715 g^3)))    (picolm/tensor.c:3317-3323)
template <int ACT> __device__ __forceinline__ float gate_act(float g);
template <> __device__ __forceinline__ float gate_act<0>(float g) { return g / (1.0f + expf(-g)); }
template <> __device__ __forceinline__ float gate_act<1>(float g) {
    return 0.5f * g * (1.0f + tanhf(0.79788456f * (g + 0.044715f * g * g * g)));
}
template <> __device__ __forceinline__ float gate_act<2>(float g) { return g; }       // (ACT 2 takes both branches: gate_clamped)

// ACT 2: both branches clamped, a sigmoid gate with a slope, and the up branch shifted by one:
//        g' = min(g, limit), u' = clamp(u, -limit, limit), out = g' sigmoid(slope g') (u' + 1)
__device__ __forceinline__ float gate_clamped(float g, float u, float limit, float slope) {
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    return g / (1.0f + expf(-slope * g)) * (u + 1.0f);
}

template <typename T, int ACT>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, int F, size_t total, float limit, float slope) {
    pdl_launch_dependents();
    pdl_wait();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < total; i += stride) {
        const size_t t = i / F;
        const int c = (int)(i - t * F);
        const float g = to_f32<T>(gu[t * 2 * F + c]);
        const float u = to_f32<T>(gu[t * 2 * F + F + c]);
        if constexpr (ACT == 2) out[i] = from_f32<T>(gate_clamped(g, u, limit, slope));
        else out[i] = from_f32<T>(gate_act<ACT>(g) * u);
    }
}

template <typename T>
static int launch_gated(int act, int blocks, cudaStream_t stream, const T* gu, T* out, int F, size_t total, float limit,
                        float slope) {
    if (act == 0) return plm_status_of(launch_pdl(swiglu_kernel<T, 0>, blocks, 256, 0, stream, gu, out, F, total, 0.f, 0.f));
    if (act == 1) return plm_status_of(launch_pdl(swiglu_kernel<T, 1>, blocks, 256, 0, stream, gu, out, F, total, 0.f, 0.f));
    if (act == 2) return plm_status_of(launch_pdl(swiglu_kernel<T, 2>, blocks, 256, 0, stream, gu, out, F, total, limit, slope));
    return PLM_ERR_UNSUPPORTED;
}

// act: 0 silu, 1 gelu (tanh form), 2 clamped branches with a sloped sigmoid gate (`limit`, `slope`)
extern "C" int plm_swiglu(const void* gu, void* out, int dtype, int act, int n_rows, int F, float limit, float slope,
                          cudaStream_t stream) {
    if (n_rows <= 0) return PLM_OK;
    if (F <= 0) return PLM_ERR_SHAPE;
    const size_t total = (size_t)n_rows * F;
    int blocks = (int)((total + 255) / 256);
    if (blocks > PLM_SM_COUNT * 16) blocks = PLM_SM_COUNT * 16;
    if (dtype == PLM_F32) return launch_gated<float>(act, blocks, stream, (const float*)gu, (float*)out, F, total, limit, slope);
    if (dtype == PLM_BF16) return launch_gated<bf16>(act, blocks, stream, (const bf16*)gu, (bf16*)out, F, total, limit, slope);
    return PLM_ERR_DTYPE;
}

// ------------------------------------------------- RoPE + write into the cache
// qkv is [T, (H + 2G) * hd]: H query heads, then G key heads, then G value heads.
// Query heads are rotated into q_out [T, H, hd]; key heads are rotated and
// written, value heads copied, into the paged cache
//   cache[page][g][slot_in_page][hd],  page = block_table[seq][pos / PLM_PAGE].
// cos/sin are [table_len, rot_dim/2] fp32 tables; null tables mean no rotation.
// pairing 0: (x[i], x[i + rot_dim/2]); pairing 1: (x[2i], x[2i+1]).  Elements at
// and beyond rot_dim pass through.  store = 0 skips the cache (a layer that reads
// another layer's cache).
template <typename Ta, typename Tc>
__global__ void rope_store_kernel(const Ta* __restrict__ qkv, Ta* __restrict__ q_out, Tc* __restrict__ kc,
                                  Tc* __restrict__ vc, const float* __restrict__ cos_t,
                                  const float* __restrict__ sin_t, const int* __restrict__ tok_pos,
                                  const int* __restrict__ tok_seq, const int* __restrict__ block_table,
                                  int max_pages, int H, int G, int hd, int rot_dim, int pairing, int store) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int pos = PLM_POSITION(tok_pos[t]);
    const int half = hd / 2, rot_half = rot_dim / 2;
    const int n_heads = H + 2 * G;
    const Ta* row = qkv + (size_t)t * n_heads * hd;
    size_t page_base = 0;
    int in_page = 0;
    bool have_page = false;
    if (store) {
        const int page = PLM_PAGE_NO(block_table[(size_t)PLM_SEQ_NO(tok_seq[t]) * max_pages + pos / PLM_PAGE]);
        have_page = page >= 0;
        page_base = (size_t)(page < 0 ? 0 : page) * G;
        in_page = pos % PLM_PAGE;
    }
    for (int item = blockIdx.y * blockDim.x + threadIdx.x; item < n_heads * half; item += gridDim.y * blockDim.x) {
        const int head = item / half, j = item - head * half;
        int ia, ib;
        bool rotate = (j < rot_half) && cos_t != nullptr;
        if (j < rot_half) {
            if (pairing == 0) { ia = j; ib = j + rot_half; } else { ia = 2 * j; ib = 2 * j + 1; }
        } else {
            ia = rot_dim + 2 * (j - rot_half); ib = ia + 1;
        }
        float a = to_f32<Ta>(row[head * hd + ia]);
        float b = to_f32<Ta>(row[head * hd + ib]);
        if (head < H) {
            if (rotate) {
                const float c = cos_t[(size_t)pos * rot_half + j], s = sin_t[(size_t)pos * rot_half + j];
                const float ra = rope_first(a, b, c, s), rb = rope_second(a, b, c, s);
                a = ra; b = rb;
            }
            Ta* o = q_out + ((size_t)t * H + head) * hd;
            o[ia] = from_f32<Ta>(a);
            o[ib] = from_f32<Ta>(b);
        } else if (head < H + G) {
            if (!store || !have_page) continue;
            if (rotate) {
                const float c = cos_t[(size_t)pos * rot_half + j], s = sin_t[(size_t)pos * rot_half + j];
                const float ra = rope_first(a, b, c, s), rb = rope_second(a, b, c, s);
                a = ra; b = rb;
            }
            const int g = head - H;
            Tc* o = kc + ((page_base + g) * PLM_PAGE + in_page) * hd;
            o[ia] = from_f32<Tc>(a);
            o[ib] = from_f32<Tc>(b);
        } else {
            if (!store || !have_page) continue;
            const int g = head - H - G;
            Tc* o = vc + ((page_base + g) * PLM_PAGE + in_page) * hd;
            o[ia] = from_f32<Tc>(a);
            o[ib] = from_f32<Tc>(b);
        }
    }
}

// The common case eight pairs at a time: bf16, the whole head rotated (rot_dim == hd), half-split
// pairing, head size a multiple of 16.  A thread takes x[j..j+8) and x[half+j..half+j+8) of one head
// as two 16-byte loads and writes two 16-byte stores.
__global__ void rope_store_vec_kernel(const bf16* __restrict__ qkv, bf16* __restrict__ q_out, bf16* __restrict__ kc,
                                      bf16* __restrict__ vc, const float* __restrict__ cos_t,
                                      const float* __restrict__ sin_t, const int* __restrict__ tok_pos,
                                      const int* __restrict__ tok_seq, const int* __restrict__ block_table,
                                      int max_pages, int H, int G, int hd, int store) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int pos = PLM_POSITION(tok_pos[t]);
    const int half = hd / 2, groups = half / 8;
    const int n_heads = H + 2 * G;
    const bf16* row = qkv + (size_t)t * n_heads * hd;
    size_t page_base = 0;
    int in_page = 0;
    bool have_page = false;
    if (store) {
        const int page = PLM_PAGE_NO(block_table[(size_t)PLM_SEQ_NO(tok_seq[t]) * max_pages + pos / PLM_PAGE]);
        have_page = page >= 0;
        page_base = (size_t)(page < 0 ? 0 : page) * G;
        in_page = pos % PLM_PAGE;
    }
    for (int item = blockIdx.y * blockDim.x + threadIdx.x; item < n_heads * groups; item += gridDim.y * blockDim.x) {
        const int head = item / groups, j = (item - head * groups) * 8;
        bf16* dst;
        if (head < H) {
            dst = q_out + ((size_t)t * H + head) * hd;
        } else {
            if (!store || !have_page) continue;
            const int g = head < H + G ? head - H : head - H - G;
            dst = (head < H + G ? kc : vc) + ((page_base + g) * PLM_PAGE + in_page) * hd;
        }
        uint4 lo = *reinterpret_cast<const uint4*>(row + head * hd + j);
        uint4 hi = *reinterpret_cast<const uint4*>(row + head * hd + half + j);
        if (head < H + G) {
            const float4 c0 = load4(cos_t + (size_t)pos * half + j), c1 = load4(cos_t + (size_t)pos * half + j + 4);
            const float4 s0 = load4(sin_t + (size_t)pos * half + j), s1 = load4(sin_t + (size_t)pos * half + j + 4);
            const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
            const float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
            __nv_bfloat162* l2 = reinterpret_cast<__nv_bfloat162*>(&lo);
            __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&hi);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float a0 = __low2float(l2[k]), a1 = __high2float(l2[k]);
                const float b0 = __low2float(h2[k]), b1 = __high2float(h2[k]);
                l2[k] = __floats2bfloat162_rn(rope_first(a0, b0, c[2 * k], sn[2 * k]), rope_first(a1, b1, c[2 * k + 1], sn[2 * k + 1]));
                h2[k] = __floats2bfloat162_rn(rope_second(a0, b0, c[2 * k], sn[2 * k]), rope_second(a1, b1, c[2 * k + 1], sn[2 * k + 1]));
            }
        }
        *reinterpret_cast<uint4*>(dst + j) = lo;
        *reinterpret_cast<uint4*>(dst + half + j) = hi;
    }
}

extern "C" int plm_rope_store(const void* qkv, void* q_out, void* kc, void* vc, int dtype, const float* cos_t,
                              const float* sin_t, const int* tok_pos, const int* tok_seq, const int* block_table,
                              int max_pages, int n_tokens, int H, int G, int hd, int rot_dim, int pairing, int store,
                              cudaStream_t stream) {
    if (n_tokens <= 0) return PLM_OK;
    if (H <= 0 || G <= 0 || hd <= 0 || (hd & 1) || rot_dim < 0 || rot_dim > hd || (rot_dim & 1)) return PLM_ERR_SHAPE;
    if (pairing != 0 && pairing != 1) return PLM_ERR_UNSUPPORTED;
    if (dtype == PLM_BF16 && pairing == 0 && rot_dim == hd && hd % 16 == 0 && cos_t != nullptr) {
        const int vitems = (H + 2 * G) * (hd / 16);
        int vchunks = (vitems + 127) / 128;
        if (vchunks > 64) vchunks = 64;
        return plm_status_of(launch_pdl(rope_store_vec_kernel, dim3(n_tokens, vchunks), dim3(128), 0, stream,
                                        (const bf16*)qkv, (bf16*)q_out, (bf16*)kc, (bf16*)vc, cos_t, sin_t, tok_pos,
                                        tok_seq, block_table, max_pages, H, G, hd, store));
    }
    const int items = (H + 2 * G) * (hd / 2);
    const int nt_threads = items >= 128 ? 128 : 64;
    int chunks = (items + nt_threads - 1) / nt_threads;
    if (chunks > 64) chunks = 64;
    const dim3 nt(nt_threads), grid_rs(n_tokens, chunks);
    if (dtype == PLM_F32)
        return plm_status_of(launch_pdl(rope_store_kernel<float, float>, grid_rs, nt, 0, stream, (const float*)qkv,
                                        (float*)q_out, (float*)kc, (float*)vc, cos_t, sin_t, tok_pos,
                                        tok_seq, block_table, max_pages, H, G, hd, rot_dim, pairing, store));
    if (dtype == PLM_BF16)
        return plm_status_of(launch_pdl(rope_store_kernel<bf16, bf16>, grid_rs, nt, 0, stream, (const bf16*)qkv,
                                        (bf16*)q_out, (bf16*)kc, (bf16*)vc, cos_t, sin_t, tok_pos,
                                        tok_seq, block_table, max_pages, H, G, hd, rot_dim, pairing, store));
    return PLM_ERR_DTYPE;
}

// dst[i, :] = src[rows[i], :] for rows of `row_bytes` bytes (a multiple of 4; 16 bytes at a time where the rows
// and both pointers allow it).  Rows of a prompt step that are wanted further on, out of all of its rows.
__global__ void gather_rows_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, const int* __restrict__ rows,
                                   long row_bytes, long src_ld, int wide) {
    pdl_launch_dependents();
    pdl_wait();
    const int i = blockIdx.x;
    const uint8_t* s = src + (size_t)PLM_ROW_NO(rows[i]) * src_ld;
    uint8_t* d = dst + (size_t)i * row_bytes;
    if (wide) {
        for (long o = (long)threadIdx.x * 16; o < row_bytes; o += (long)blockDim.x * 16)
            *reinterpret_cast<uint4*>(d + o) = *reinterpret_cast<const uint4*>(s + o);
    } else {
        for (long o = (long)threadIdx.x * 4; o < row_bytes; o += (long)blockDim.x * 4)
            *reinterpret_cast<uint32_t*>(d + o) = *reinterpret_cast<const uint32_t*>(s + o);
    }
}

extern "C" int plm_gather_rows(const void* src, void* dst, const int* rows, int n_rows, long row_bytes, long src_ld_bytes,
                               cudaStream_t stream) {
    if (n_rows <= 0 || row_bytes <= 0) return PLM_OK;
    if (row_bytes % 4 || src_ld_bytes % 4 || (((uintptr_t)src | (uintptr_t)dst) & 3)) return PLM_ERR_ALIGN;
    const int wide = row_bytes % 16 == 0 && src_ld_bytes % 16 == 0 && ((((uintptr_t)src | (uintptr_t)dst) & 15) == 0);
    return plm_status_of(launch_pdl(gather_rows_kernel, dim3(n_rows), dim3(256), 0, stream, (const uint8_t*)src,
                                    (uint8_t*)dst, rows, row_bytes, src_ld_bytes, wide));
}

// ------------------------------------------------------------------ layer norm
// out = (v - mean) / sqrt(var + eps) * w with v = x (+ delta) (+ bias), mean and var (the mean squared deviation
// from the mean) over the row, no bias after the weight.  One block per output row, like the RMSNorm above: row r
// reads source row rows[r] (or r); with a delta or a bias the sum is written back to x unless rows are gathered.
// `bias` [d] fp32 is a projection's bias that its product left out (a product's epilogue adds no bias).  The row
// stays in shared memory between the passes (mean, deviations, output), so x is read once.
template <typename Tw, typename To, int NT>
__global__ void __launch_bounds__(NT)
layernorm_kernel(float* __restrict__ x, const float* __restrict__ delta, const float* __restrict__ bias,
                 const Tw* __restrict__ w, To* __restrict__ out, const int* __restrict__ rows, int d, float eps,
                 int write_back) {
    extern __shared__ float row_sm[];               // [d]
    __shared__ float red[33];
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    const int src = rows ? PLM_ROW_NO(rows[r]) : r;
    float* xr = x + (size_t)src * d;
    const float* dr = delta ? delta + (size_t)src * d : nullptr;
    float s = 0.f;
    for (int i = threadIdx.x; i < d; i += NT) {
        float v = xr[i];
        if (dr) v += dr[i];
        if (bias) v += bias[i];
        if (write_back) xr[i] = v;
        row_sm[i] = v;
        s += v;
    }
    const float mean = block_sum<NT>(s, red) / (float)d;
    float ss = 0.f;
    for (int i = threadIdx.x; i < d; i += NT) {
        const float c = row_sm[i] - mean;
        ss += c * c;
    }
    ss = block_sum<NT>(ss, red);
    const float scale = 1.0f / sqrtf(ss / (float)d + eps);
    To* o = out + (size_t)r * d;
    for (int i = threadIdx.x; i < d; i += NT) o[i] = from_f32<To>((row_sm[i] - mean) * scale * to_f32<Tw>(w[i]));
}

// Four elements at a time, the row kept in registers between the passes: for rows whose width is a multiple of 4 and
// at most 16 * NT (and 16-byte aligned pointers).
template <typename Tw, typename To, int NT>
__global__ void __launch_bounds__(NT)
layernorm_vec_kernel(float* __restrict__ x, const float* __restrict__ delta, const float* __restrict__ bias,
                     const Tw* __restrict__ w, To* __restrict__ out, const int* __restrict__ rows, int d, float eps,
                     int write_back) {
    __shared__ float red[33];
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    const int src = rows ? PLM_ROW_NO(rows[r]) : r;
    float* xr = x + (size_t)src * d;
    const float* dr = delta ? delta + (size_t)src * d : nullptr;
    float4 v[4];
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int i = (threadIdx.x + k * NT) * 4;
        if (i < d) {
            v[k] = load4(xr + i);
            if (dr) {
                const float4 dv = load4(dr + i);
                v[k].x += dv.x; v[k].y += dv.y; v[k].z += dv.z; v[k].w += dv.w;
            }
            if (bias) {
                const float4 bv = load4(bias + i);
                v[k].x += bv.x; v[k].y += bv.y; v[k].z += bv.z; v[k].w += bv.w;
            }
            if (write_back) store4(xr + i, v[k]);
            s += (v[k].x + v[k].y) + (v[k].z + v[k].w);
        }
    }
    const float mean = block_sum<NT>(s, red) / (float)d;
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int i = (threadIdx.x + k * NT) * 4;
        if (i < d) {
            v[k].x -= mean; v[k].y -= mean; v[k].z -= mean; v[k].w -= mean;
            ss += v[k].x * v[k].x + v[k].y * v[k].y + v[k].z * v[k].z + v[k].w * v[k].w;
        }
    }
    ss = block_sum<NT>(ss, red);
    const float scale = 1.0f / sqrtf(ss / (float)d + eps);
    To* o = out + (size_t)r * d;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int i = (threadIdx.x + k * NT) * 4;
        if (i < d) {
            const float4 wv = load4(w + i);
            store4(o + i, make_float4(v[k].x * scale * wv.x, v[k].y * scale * wv.y, v[k].z * scale * wv.z, v[k].w * scale * wv.w));
        }
    }
}

template <typename Tw, typename To>
static int layernorm_launch(float* x, const float* delta, const float* bias, const void* w, void* out, const int* rows,
                            int n_rows, int d, float eps, int write_back, cudaStream_t stream) {
    // the kernel and the block size (and with them the order of the sums) depend on the row's width only
    if (d % 4 == 0 && d <= 16 * 1024 && ((((uintptr_t)x | (uintptr_t)delta | (uintptr_t)bias | (uintptr_t)w | (uintptr_t)out) & 15) == 0)) {
        if (d <= 16 * 256)
            return plm_status_of(launch_pdl(layernorm_vec_kernel<Tw, To, 256>, n_rows, 256, 0, stream, x, delta, bias, (const Tw*)w,
                                            (To*)out, rows, d, eps, write_back));
        return plm_status_of(launch_pdl(layernorm_vec_kernel<Tw, To, 1024>, n_rows, 1024, 0, stream, x, delta, bias, (const Tw*)w,
                                        (To*)out, rows, d, eps, write_back));
    }
    const size_t smem = (size_t)d * sizeof(float);
    if (d > 1024) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(layernorm_kernel<Tw, To, 1024>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        return plm_status_of(launch_pdl(layernorm_kernel<Tw, To, 1024>, n_rows, 1024, smem, stream, x, delta, bias,
                                        (const Tw*)w, (To*)out, rows, d, eps, write_back));
    }
    return plm_status_of(launch_pdl(layernorm_kernel<Tw, To, 256>, n_rows, 256, smem, stream, x, delta, bias, (const Tw*)w,
                                    (To*)out, rows, d, eps, write_back));
}

extern "C" int plm_layernorm(float* x, const float* delta, const float* bias, const void* w, int w_dtype, void* out,
                             int out_dtype, const int* rows, int n_rows, int d, float eps, cudaStream_t stream) {
    if (n_rows <= 0) return PLM_OK;
    if (d <= 0 || d > 56 * 1024) return PLM_ERR_SHAPE;
    const int write_back = ((delta != nullptr || bias != nullptr) && rows == nullptr) ? 1 : 0;
    if (w_dtype == PLM_F32 && out_dtype == PLM_F32)
        return layernorm_launch<float, float>(x, delta, bias, w, out, rows, n_rows, d, eps, write_back, stream);
    if (w_dtype == PLM_BF16 && out_dtype == PLM_F32)
        return layernorm_launch<bf16, float>(x, delta, bias, w, out, rows, n_rows, d, eps, write_back, stream);
    if (w_dtype == PLM_F32 && out_dtype == PLM_BF16)
        return layernorm_launch<float, bf16>(x, delta, bias, w, out, rows, n_rows, d, eps, write_back, stream);
    if (w_dtype == PLM_BF16 && out_dtype == PLM_BF16)
        return layernorm_launch<bf16, bf16>(x, delta, bias, w, out, rows, n_rows, d, eps, write_back, stream);
    return PLM_ERR_DTYPE;
}

// x[t, :] += bias[:] in place on fp32 rows: a projection's bias, where nothing that follows can take it along.
__global__ void add_bias_kernel(float* __restrict__ x, const float* __restrict__ bias, int d, size_t total) {
    pdl_launch_dependents();
    pdl_wait();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < total; i += stride) x[i] += bias[i % d];
}

extern "C" int plm_add_bias(float* x, const float* bias, int n_rows, int d, cudaStream_t stream) {
    if (n_rows <= 0) return PLM_OK;
    if (d <= 0) return PLM_ERR_SHAPE;
    const size_t total = (size_t)n_rows * d;
    int blocks = (int)((total + 255) / 256);
    if (blocks > PLM_SM_COUNT * 16) blocks = PLM_SM_COUNT * 16;
    return plm_status_of(launch_pdl(add_bias_kernel, dim3(blocks), dim3(256), 0, stream, x, bias, d, total));
}

// ------------------------- bias + norm over the whole projection + RoPE + write into the cache
// What stands between the QKV product and attention in a layer whose queries and keys are normalised over ALL
// heads at once before they are rotated.  qkv is [T, nq + nk + nv] with nq = H * D query columns, then (a layer
// that keeps keys and values of its own: own_kv) nk = G * D key columns and nv = G * Dv value columns; keys and
// values may differ in width.  Per token, in fp32:
//   q += bias_q; q *= 1 / sqrt(mean(q^2 over all nq columns) + eps) * wq;   the same for k with wk (null weights: no norm)
//   the leading rot_dim components of every head of q and k are rotated by the token's position
//   (pairing 0: (x[i], x[i + rot_dim/2]); pairing 1: (x[2i], x[2i+1])), the others pass
//   v += bias_v
// Queries go to q_out [T, H, hd_c], keys and values into the paged cache [pages, G, PLM_PAGE, hd_c]; hd_c >= D, Dv
// is the one head size of the cache and of the attention kernels, and what lies beyond a head's own width is
// written as zero (a zero component adds nothing to a score; a zero value column is multiplied by zero weights of
// the output projection).  One block per token; the token's q and k sit in shared memory between the sums of
// squares and the rotation; sums in an order that depends on the sizes only.  A row of qkv is ld elements long (the
// product may hold further columns, a gate's for instance, behind q, k and v); q_scale [H] (or null) multiplies head
// h's queries after norm and rotation: a factor per head on its scores.
__device__ __forceinline__ void store_pair(float* p, float a, float b) { *reinterpret_cast<float2*>(p) = make_float2(a, b); }
__device__ __forceinline__ void store_pair(bf16* p, float a, float b) { *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b); }

template <typename Ta, typename Tw, typename Tc, int NT, bool CONV>
__global__ void __launch_bounds__(NT)
qk_norm_rope_store_kernel(const Ta* __restrict__ qkv, const float* __restrict__ bias, const Tw* __restrict__ wq,
                          const Tw* __restrict__ wk, float eps, Tc* __restrict__ q_out, Tc* __restrict__ kc,
                          Tc* __restrict__ vc, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                          const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                          const int* __restrict__ block_table, int max_pages, int H, int G, int D, int Dv, int hd_c,
                          int rot_dim, int pairing, int own_kv, int per_head, int v_from_k, long ld,
                          const float* __restrict__ q_scale, const float* __restrict__ conv_w, int taps,
                          float* __restrict__ conv_state, long state_stride, const int* __restrict__ seq_start,
                          const int* __restrict__ seq_slot, int conv_keeps_state) {
    extern __shared__ float qk_sm[];                 // [nq + nk] (with a convolution: [nq + nk + nv])
    __shared__ float red[33];
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    // v_from_k: there is no value projection; the keys as projected (with their bias, before norm and rotation) are the values
    const int nq = H * D, nk = own_kv ? G * D : 0, nv = own_kv && !v_from_k ? G * Dv : 0;
    const int pos = PLM_POSITION(tok_pos[t]);
    const Ta* row = qkv + (size_t)t * ld;           // (ld >= nq + nk + nv: the product may hold more columns behind them)
    // conv_w [taps][nq + nk + nv] (tap-major, the token's own tap last): every column is first convolved over time with
    // the projected rows of the sequence's tokens before, which lie in the rows above this one or, for tokens before the
    // step's first, in conv_state [slot][taps - 1][columns] (oldest first).  With conv_keeps_state (a step of one token a
    // sequence) the thread that reads a column's state also moves it on; otherwise a kernel of its own does that afterwards.
    const int n_cols = nq + nk + nv;
    int in_seq = 0;
    float* conv_st = nullptr;
    if (CONV) {
        const int b = PLM_SEQ_NO(tok_seq[t]);
        in_seq = t - seq_start[b];
        conv_st = conv_state + (long)seq_slot[b] * state_stride;
    }
    auto column = [&](int c) -> float {
        if (!CONV) return to_f32<Ta>(row[c]);
        float acc = 0.f;
        if (taps <= 8) {
            // all taps' inputs asked for at once, then the sum in the same order
            float u[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int back = taps - 1 - j, li = in_seq - back;
                u[j] = 0.f;
                if (j < taps) u[j] = li >= 0 ? to_f32<Ta>(qkv[(size_t)(t - back) * ld + c]) : conv_st[(long)(taps - 1 + li) * n_cols + c];
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                if (j < taps) {
                    acc = fmaf(conv_w[(long)j * n_cols + c], u[j], acc);
                    if (conv_keeps_state && j > 0) conv_st[(long)(j - 1) * n_cols + c] = u[j];
                }
            }
            return acc;
        }
        for (int j = 0; j < taps; ++j) {
            const int back = taps - 1 - j, li = in_seq - back;
            const float u = li >= 0 ? to_f32<Ta>(qkv[(size_t)(t - back) * ld + c]) : conv_st[(long)(taps - 1 + li) * n_cols + c];
            acc = fmaf(conv_w[(long)j * n_cols + c], u, acc);
            if (conv_keeps_state && j > 0) conv_st[(long)(j - 1) * n_cols + c] = u;
        }
        return acc;
    };
    float sq = 0.f, sk = 0.f;
    const bool batched = CONV && taps <= 4;          // (then the values' columns are convolved here too, into shared memory)
    if (batched) {
        // four of a thread's columns at a time: all their taps' inputs are asked for before any is used (a thread's
        // columns in ascending order, as below, so the sums of squares keep their order)
        const bool above = in_seq >= taps - 1;       // every input lies in the step's rows above
        for (int i0 = threadIdx.x; i0 < n_cols; i0 += NT * 4) {
            float u[4][4];
#pragma unroll
            for (int m = 0; m < 4; ++m) {
                const int c = i0 + m * NT;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int back = taps - 1 - j, li = in_seq - back;
                    u[m][j] = 0.f;
                    if (c < n_cols && j < taps)
                        u[m][j] = (above || li >= 0) ? to_f32<Ta>(row[c - (long)back * ld]) : conv_st[(taps - 1 + li) * n_cols + c];
                }
            }
#pragma unroll
            for (int m = 0; m < 4; ++m) {
                const int c = i0 + m * NT;
                if (c >= n_cols) continue;
                float acc = 0.f;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    if (j < taps) {
                        acc = fmaf(conv_w[j * n_cols + c], u[m][j], acc);
                        if (conv_keeps_state && j > 0) conv_st[(j - 1) * n_cols + c] = u[m][j];
                    }
                }
                qk_sm[c] = acc;
                if (c < nq) sq += acc * acc; else if (c < nq + nk) sk += acc * acc;
            }
        }
    } else
    for (int i = threadIdx.x; i < nq + nk; i += NT) {
        float v = column(i);
        if (bias) v += bias[i];
        qk_sm[i] = v;
        if (i < nq) sq += v * v; else sk += v * v;
    }
    sq = block_sum<NT>(sq, red);
    // per_head: the root mean square is taken over each head's own D columns (below), the weight [D] serves every head
    const float rq = wq && !per_head ? 1.0f / sqrtf(sq / (float)nq + eps) : 1.0f;
    float rk = 1.0f;
    if (nk > 0) {
        sk = block_sum<NT>(sk, red);
        if (wk && !per_head) rk = 1.0f / sqrtf(sk / (float)nk + eps);
    }
    size_t page_base = 0;
    int in_page = 0;
    bool have_page = false;
    if (own_kv) {
        const int page = PLM_PAGE_NO(block_table[(size_t)PLM_SEQ_NO(tok_seq[t]) * max_pages + pos / PLM_PAGE]);
        have_page = page >= 0;
        page_base = (size_t)(page < 0 ? 0 : page) * G;
        in_page = pos % PLM_PAGE;
    }
    const int rot_half = rot_dim / 2, half_c = hd_c / 2;
    const int heads = H + (own_kv ? G : 0);
    // pairs of output components (ia, ib) of a head of hd_c: the rotated pairs first, then neighbours.  A warp takes a
    // head, its lanes the head's pairs (no division a pair); neighbours are written as one 4- or 8-byte store.
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const float* cos_p = cos_t ? cos_t + (size_t)pos * rot_half : nullptr;
    const float* sin_p = cos_t ? sin_t + (size_t)pos * rot_half : nullptr;
    for (int head = warp; head < heads; head += NT / 32) {
        const bool is_q = head < H;
        const int hh = is_q ? head : head - H;
        const float* src = qk_sm + (is_q ? 0 : nq) + hh * D;
        const Tw* wn = is_q ? wq : wk;
        if (wn && !per_head) wn += hh * D;
        float r = is_q ? rq : rk;
        if (wn && per_head) {
            float ss = 0.f;
            for (int j = lane; j < D; j += 32) ss = fmaf(src[j], src[j], ss);
            r = 1.0f / sqrtf(warp_sum(ss) / (float)D + eps);
        }
        // a factor per query head on its scores: the query carries it (a rotation does not change it)
        const float hs = is_q && q_scale ? q_scale[hh] : 1.0f;
        Tc* o;
        if (is_q) {
            o = q_out + ((size_t)t * H + hh) * hd_c;
        } else {
            if (!have_page) continue;
            o = kc + ((page_base + hh) * PLM_PAGE + in_page) * hd_c;
        }
        for (int j = lane; j < half_c; j += 32) {
            int ia, ib;
            const bool rotate = j < rot_half && cos_p != nullptr;
            if (j < rot_half) {
                if (pairing == 0) { ia = j; ib = j + rot_half; } else { ia = 2 * j; ib = 2 * j + 1; }
            } else {
                ia = rot_dim + 2 * (j - rot_half); ib = ia + 1;
            }
            float a = 0.f, b = 0.f;
            if (ia < D) { a = src[ia]; if (wn) a = a * r * to_f32<Tw>(wn[ia]); }
            if (ib < D) { b = src[ib]; if (wn) b = b * r * to_f32<Tw>(wn[ib]); }
            if (rotate) {
                const float c = cos_p[j], s = sin_p[j];
                const float ra = rope_first(a, b, c, s), rb = rope_second(a, b, c, s);
                a = ra; b = rb;
            }
            a *= hs; b *= hs;
            if (ib == ia + 1) {
                store_pair(o + ia, a, b);
            } else {
                o[ia] = from_f32<Tc>(a);
                o[ib] = from_f32<Tc>(b);
            }
        }
    }
    if (own_kv && have_page) {
        for (int item = threadIdx.x; item < G * hd_c; item += NT) {
            const int g = item / hd_c, c = item - g * hd_c;
            float v = 0.f;
            if (v_from_k) {
                if (c < D) v = qk_sm[nq + g * D + c];
            } else if (c < Dv) {
                v = batched ? qk_sm[nq + nk + g * Dv + c] : column(nq + nk + g * Dv + c);
                if (bias) v += bias[nq + nk + g * Dv + c];
            }
            vc[((page_base + g) * PLM_PAGE + in_page) * hd_c + c] = from_f32<Tc>(v);
        }
    }
}

// The convolution's tail after a step of several tokens a sequence: the last taps - 1 projected rows of every sequence,
// oldest first (old tail rows move up where the step brought fewer).  One thread per (sequence, column); it reads what
// it needs of the old tail before it writes (ascending s: slot s takes old slot s + n > s).
template <typename Ta>
__global__ void conv_tail_kernel(const Ta* __restrict__ qkv, long ld, float* __restrict__ state, long state_stride,
                                 const int* __restrict__ seq_start, const int* __restrict__ seq_slot, int n_seqs, int C, int taps) {
    pdl_launch_dependents();
    pdl_wait();
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long)n_seqs * C) return;
    const int b = (int)(idx / C), c = (int)(idx % C);
    const int t0 = seq_start[b], n = seq_start[b + 1] - t0;
    if (n <= 0) return;
    float* st = state + (long)seq_slot[b] * state_stride;
    for (int s = 0; s < taps - 1; ++s) {
        const int src = n - (taps - 1) + s;
        st[(long)s * C + c] = src >= 0 ? to_f32<Ta>(qkv[(size_t)(t0 + src) * ld + c]) : st[(long)(s + n) * C + c];
    }
}

// qkv_dtype: the projection's result (PLM_F32, or PLM_BF16); out_dtype: queries, cache and norm weights.
extern "C" int plm_qk_norm_rope_store(const void* qkv, int qkv_dtype, const float* bias, const void* wq, const void* wk,
                                      float eps, void* q_out, void* kc, void* vc, int out_dtype, const float* cos_t,
                                      const float* sin_t, const int* tok_pos, const int* tok_seq, const int* block_table,
                                      int max_pages, int n_tokens, int H, int G, int D, int Dv, int hd_c, int rot_dim,
                                      int pairing, int own_kv, int per_head, int v_from_k, long ld, const float* q_scale,
                                      const float* conv_w, int taps, float* conv_state, long state_stride,
                                      const int* seq_start, const int* seq_slot, int n_seqs, int one_token_each,
                                      cudaStream_t stream) {
    if (n_tokens <= 0) return PLM_OK;
    const int conv_cols = H * D + (own_kv ? G * D + (v_from_k ? 0 : G * Dv) : 0);
    if (conv_w != nullptr && (taps < 1 || bias != nullptr || (taps > 1 && (conv_state == nullptr || seq_start == nullptr ||
        seq_slot == nullptr || n_seqs <= 0 || state_stride < (long)(taps - 1) * conv_cols))))
        return PLM_ERR_SHAPE;
    // one token a sequence: the block that reads a sequence's tail also writes it
    const int conv_keeps_state = conv_w != nullptr && one_token_each && n_seqs == n_tokens ? 1 : 0;
    if (ld < (long)H * D + (own_kv ? (long)G * D + (v_from_k ? 0 : (long)G * Dv) : 0)) return PLM_ERR_SHAPE;
    if (H <= 0 || G <= 0 || D <= 0 || Dv <= 0 || hd_c < D || hd_c < Dv || (hd_c & 1) || rot_dim < 0 || rot_dim > D ||
        (rot_dim & 1))
        return PLM_ERR_SHAPE;
    if (pairing != 0 && pairing != 1) return PLM_ERR_UNSUPPORTED;
    const size_t smem = (size_t)(conv_w ? conv_cols : H * D + (own_kv ? G * D : 0)) * sizeof(float);
    if (smem > 200 * 1024) return PLM_ERR_SHAPE;
#define QKN_LAUNCH(Ta_, Tc_)                                                                                           \
    do {                                                                                                               \
        if (smem > 48 * 1024)                                                                                          \
            cudaFuncSetAttribute(conv_w ? qk_norm_rope_store_kernel<Ta_, Tc_, Tc_, 256, true> : qk_norm_rope_store_kernel<Ta_, Tc_, Tc_, 256, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        cudaError_t e_ = launch_pdl(conv_w ? qk_norm_rope_store_kernel<Ta_, Tc_, Tc_, 256, true> : qk_norm_rope_store_kernel<Ta_, Tc_, Tc_, 256, false>, dim3(n_tokens), dim3(256), smem, stream, \
                                        (const Ta_*)qkv, bias, (const Tc_*)wq, (const Tc_*)wk, eps, (Tc_*)q_out, (Tc_*)kc, \
                                        (Tc_*)vc, cos_t, sin_t, tok_pos, tok_seq, block_table, max_pages, H, G, D, Dv,  \
                                        hd_c, rot_dim, pairing, own_kv, per_head, v_from_k, ld, q_scale, conv_w, taps,  \
                                        conv_state, state_stride, seq_start, seq_slot, conv_keeps_state);              \
        if (e_ != cudaSuccess || conv_w == nullptr || taps == 1 || conv_keeps_state) return plm_status_of(e_);         \
        return plm_status_of(launch_pdl(conv_tail_kernel<Ta_>, dim3((unsigned)(((long)n_seqs * conv_cols + 255) / 256)), \
                                        dim3(256), 0, stream, (const Ta_*)qkv, ld, conv_state, state_stride, seq_start, \
                                        seq_slot, n_seqs, conv_cols, taps));                                           \
    } while (0)
    if (qkv_dtype == PLM_F32 && out_dtype == PLM_F32) QKN_LAUNCH(float, float);
    if (qkv_dtype == PLM_F32 && out_dtype == PLM_BF16) QKN_LAUNCH(float, bf16);
    if (qkv_dtype == PLM_BF16 && out_dtype == PLM_BF16) QKN_LAUNCH(bf16, bf16);
#undef QKN_LAUNCH
    return PLM_ERR_DTYPE;
}


// ------------------------------------------------------------------------------------------------ Dynamic Tanh
// A norm without statistics: out = tanh(alpha * v) * w + b, elementwise, v = x (+ delta (+ dbias)).  With `post_w`
// the delta is first divided by its own root mean square (eps inside the root) and multiplied by post_w: a
// sublayer's result that is normalised before it is added.  The sum is written back to x unless rows are gathered.
__device__ __forceinline__ float gelu_tanh_f(float z) {
    return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

template <typename To, int NT>
__global__ void __launch_bounds__(NT)
dyt_norm_kernel(float* __restrict__ x, const float* __restrict__ delta, const float* __restrict__ dbias,
                const float* __restrict__ post_w, float post_eps, const float* __restrict__ extra,
                const float* __restrict__ alpha, const float* __restrict__ w, const float* __restrict__ b,
                To* __restrict__ out, const int* __restrict__ rows, int d, int write_back) {
    __shared__ float red[33];
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    const int src = rows ? PLM_ROW_NO(rows[r]) : r;
    float* xr = x + (size_t)src * d;
    const float* dr = delta ? delta + (size_t)src * d : nullptr;
    const float* er = extra ? extra + (size_t)src * d : nullptr;
    float post = 1.0f;
    if (dr && post_w) {
        float ss = 0.f;
        for (int i = threadIdx.x; i < d; i += NT) ss = fmaf(dr[i], dr[i], ss);
        post = 1.0f / sqrtf(block_sum<NT>(ss, red) / (float)d + post_eps);
    }
    const float a = alpha ? alpha[0] : 0.f;
    To* o = out ? out + (size_t)r * d : nullptr;
    for (int i = threadIdx.x; i < d; i += NT) {
        float v = xr[i];
        if (dr) v += post_w ? dr[i] * post * post_w[i] : dr[i];
        if (dbias) v += dbias[i];
        if (er) v += er[i];
        if (write_back) xr[i] = v;
        if (o) o[i] = from_f32<To>(alpha ? fmaf(tanhf(a * v), w[i], b[i]) : v);
    }
}

// v = x + delta' + dbias + extra, in that order (every addend may be null; delta' is delta, or with `post_w` delta over
// its root mean square times post_w).  The sum is written back to x unless `rows` gathers.  out (may be null) receives
// tanh(alpha v) w + b, or v itself where alpha is null.
extern "C" int plm_dyt_norm(float* x, const float* delta, const float* dbias, const float* post_w, float post_eps,
                            const float* extra, const float* alpha, const float* w, const float* b, void* out, int out_dtype,
                            const int* rows, int n_rows, int d, cudaStream_t stream) {
    if (n_rows <= 0) return PLM_OK;
    if (d <= 0) return PLM_ERR_SHAPE;
    const int write_back = rows == nullptr && (delta != nullptr || dbias != nullptr || extra != nullptr);
    if (out_dtype == PLM_F32)
        return plm_status_of(launch_pdl(dyt_norm_kernel<float, 256>, dim3(n_rows), dim3(256), 0, stream, x, delta, dbias, post_w,
                                        post_eps, extra, alpha, w, b, (float*)out, rows, d, write_back));
    if (out_dtype == PLM_BF16)
        return plm_status_of(launch_pdl(dyt_norm_kernel<bf16, 256>, dim3(n_rows), dim3(256), 0, stream, x, delta, dbias, post_w,
                                        post_eps, extra, alpha, w, b, (bf16*)out, rows, d, write_back));
    return PLM_ERR_DTYPE;
}

// x[r, :] += a[r, :] + b[r, :] + vec[:], in that order; every addend may be null.
__global__ void add_rows_kernel(float* __restrict__ x, const float* __restrict__ a, const float* __restrict__ b,
                                const float* __restrict__ vec, long n, int d) {
    pdl_launch_dependents();
    pdl_wait();
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float v = x[i];
    if (a) v += a[i];
    if (b) v += b[i];
    if (vec) v += vec[i % d];
    x[i] = v;
}

extern "C" int plm_add_rows(float* x, const float* a, const float* b, const float* vec, int n_rows, int d, cudaStream_t stream) {
    if (n_rows <= 0) return PLM_OK;
    const long n = (long)n_rows * d;
    return plm_status_of(launch_pdl(add_rows_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, x, a, b, vec, n, d));
}

// out[r, :] = sa * (a[r, :] + bias_a[:]) + sb * b[r, :]: two float32 results added with two constants.
__global__ void scaled_sum_kernel(const float* __restrict__ a, float sa, const float* __restrict__ bias_a,
                                  const float* __restrict__ b, float sb, float* __restrict__ out, long n, int d) {
    pdl_launch_dependents();
    pdl_wait();
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float va = a[i];
    if (bias_a) va += bias_a[i % d];
    out[i] = fmaf(sa, va, sb * b[i]);
}

extern "C" int plm_scaled_sum(const float* a, float sa, const float* bias_a, const float* b, float sb, float* out, int n_rows,
                              int d, cudaStream_t stream) {
    if (n_rows <= 0) return PLM_OK;
    const long n = (long)n_rows * d;
    return plm_status_of(launch_pdl(scaled_sum_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, a, sa, bias_a, b,
                                    sb, out, n, d));
}

// out[r, j] = gelu_tanh(gate[r, j]) * table[tok[row r], col0 + j]: a gate times a row of a per-token table.
template <typename T, typename Tw>
__global__ void token_gate_kernel(const T* __restrict__ gate, const Tw* __restrict__ table, long ld_table, int col0,
                                  const int* __restrict__ tok, const int* __restrict__ rows, T* __restrict__ out, int n_rows,
                                  int dim, int vocab) {
    pdl_launch_dependents();
    pdl_wait();
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long)n_rows * dim) return;
    const int r = (int)(i / dim), j = (int)(i % dim);
    int id = tok[rows ? PLM_ROW_NO(rows[r]) : r];
    id = id < 0 ? 0 : id >= vocab ? vocab - 1 : id;
    const float e = to_f32<Tw>(table[(long)id * ld_table + col0 + j]);
    out[i] = from_f32<T>(gelu_tanh_f(to_f32<T>(gate[i])) * e);
}

extern "C" int plm_token_gate(const void* gate, int dtype, const void* table, int table_dtype, long ld_table, int col0,
                              const int* tok, const int* rows, void* out, int n_rows, int dim, int vocab, cudaStream_t stream) {
    if (n_rows <= 0) return PLM_OK;
    if (dim <= 0 || vocab <= 0 || col0 < 0 || col0 + dim > ld_table) return PLM_ERR_SHAPE;
    const dim3 grid((unsigned)(((long)n_rows * dim + 255) / 256));
    if (dtype == PLM_F32 && table_dtype == PLM_F32)
        return plm_status_of(launch_pdl(token_gate_kernel<float, float>, grid, dim3(256), 0, stream, (const float*)gate,
                                        (const float*)table, ld_table, col0, tok, rows, (float*)out, n_rows, dim, vocab));
    if (dtype == PLM_BF16 && table_dtype == PLM_BF16)
        return plm_status_of(launch_pdl(token_gate_kernel<bf16, bf16>, grid, dim3(256), 0, stream, (const bf16*)gate,
                                        (const bf16*)table, ld_table, col0, tok, rows, (bf16*)out, n_rows, dim, vocab));
    return PLM_ERR_DTYPE;
}

// ------------------------------------------------------------------------------------------------ rotation in place
// x [T, n_heads, hd] with row stride ld: the leading rot_dim components of every head are rotated by the row's position
// (pairing 0: (x[i], x[i + rot_dim/2]); pairing 1: (x[2i], x[2i+1])), in fp32, in place; the others stay.  For rows that
// reach attention by another way than a QKV product (queries taken into a latent's space, for instance).
template <typename T>
__global__ void rope_rows_kernel(T* __restrict__ x, long ld, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                 const int* __restrict__ tok_pos, int n_rows, int n_heads, int hd, int rot_dim, int pairing) {
    pdl_launch_dependents();
    pdl_wait();
    const int half = rot_dim / 2;
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long)n_rows * n_heads * half) return;
    const int j = (int)(i % half);
    const long th = i / half;
    const int head = (int)(th % n_heads), t = (int)(th / n_heads);
    const int pos = PLM_POSITION(tok_pos[t]);
    T* p = x + (long)t * ld + (long)head * hd;
    const int ia = pairing == 0 ? j : 2 * j, ib = pairing == 0 ? j + half : 2 * j + 1;
    const float a = to_f32<T>(p[ia]), b = to_f32<T>(p[ib]);
    const float c = cos_t[(size_t)pos * half + j], s = sin_t[(size_t)pos * half + j];
    p[ia] = from_f32<T>(rope_first(a, b, c, s));
    p[ib] = from_f32<T>(rope_second(a, b, c, s));
}

extern "C" int plm_rope_rows(void* x, int dtype, long ld, const float* cos_t, const float* sin_t, const int* tok_pos, int n_rows,
                             int n_heads, int hd, int rot_dim, int pairing, cudaStream_t stream) {
    if (n_rows <= 0 || rot_dim == 0) return PLM_OK;
    if (n_heads <= 0 || hd <= 0 || rot_dim < 0 || (rot_dim & 1) || rot_dim > hd || ld < (long)n_heads * hd) return PLM_ERR_SHAPE;
    if (pairing != 0 && pairing != 1) return PLM_ERR_UNSUPPORTED;
    const dim3 grid((unsigned)(((long)n_rows * n_heads * (rot_dim / 2) + 255) / 256));
    if (dtype == PLM_F32)
        return plm_status_of(launch_pdl(rope_rows_kernel<float>, grid, dim3(256), 0, stream, (float*)x, ld, cos_t, sin_t, tok_pos,
                                        n_rows, n_heads, hd, rot_dim, pairing));
    if (dtype == PLM_BF16)
        return plm_status_of(launch_pdl(rope_rows_kernel<bf16>, grid, dim3(256), 0, stream, (bf16*)x, ld, cos_t, sin_t, tok_pos,
                                        n_rows, n_heads, hd, rot_dim, pairing));
    return PLM_ERR_DTYPE;
}

// ------------------------------------------------------------------------------------------------ two norms of one row
// A layer whose mixer and feed-forward read the same x through norms of their own:
//   out_a = x r w_a  (then, with `mix`, shifted towards the token before: out_a + (prev_a - out_a) * mix, where prev_a is
//           the unshifted out_a of the sequence's token before, from `state` for a step's first token; zeros at position 0)
//   out_b = x r w_b  (null: only out_a is made)
// with r = 1 / sqrt(mean(x^2) + eps), all in fp32, w_a and w_b fp32 (a weight stored around zero arrives here as 1 + w).
// One block per token; the block also works out the norm of the token before (its row of x is read once more, from the
// L2 cache as a rule: the price of needing no second pass and no meeting between blocks), unless that token lies in
// an earlier step.  `state` [slots][d] fp32 keeps each sequence's last unshifted out_a.  The sums run in an order that depends on d only, and the row before is normalised by
// the same code as the row itself, so a position's result does not depend on how the prompt was cut.
// Two sums over a block at once (the barriers of one sum instead of two); each sum's order is that of block_sum.
template <int NT>
__device__ __forceinline__ float2 block_sum2(float a, float b, float* red) {      // red: at least 66 floats
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    a = warp_sum(a);
    b = warp_sum(b);
    __syncthreads();
    if (lane == 0) { red[warp] = a; red[33 + warp] = b; }
    __syncthreads();
    if (warp == 0) {
        float ta = (lane < NT / 32) ? red[lane] : 0.f, tb = (lane < NT / 32) ? red[33 + lane] : 0.f;
        ta = warp_sum(ta);
        tb = warp_sum(tb);
        if (lane == 0) { red[32] = ta; red[65] = tb; }
    }
    __syncthreads();
    return make_float2(red[32], red[65]);
}

template <int NT>
__device__ __forceinline__ float row_sum_squares(const float* __restrict__ row, int d) {
    float ss = 0.f;
    if ((d & 3) == 0) {
        for (int i = threadIdx.x * 4; i < d; i += NT * 4) {
            const float4 v = *reinterpret_cast<const float4*>(row + i);
            ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
    } else {
        for (int i = threadIdx.x; i < d; i += NT) ss += row[i] * row[i];
    }
    return ss;
}

template <typename To, int NT>
__global__ void __launch_bounds__(NT)
norm_pair_shift_kernel(const float* __restrict__ x, const float* __restrict__ w_a, const float* __restrict__ w_b,
                       const float* __restrict__ mix, float* __restrict__ state, long state_stride,
                       const int* __restrict__ tok_seq, const int* __restrict__ seq_start, const int* __restrict__ seq_slot,
                       To* __restrict__ out_a, To* __restrict__ out_b, int d, float eps) {
    __shared__ float red[33];
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    // `other`: the row whose norm this block needs beside its own.  For a sequence's first token of the step that is the
    // sequence's LAST token of the step, whose norm goes into the state: the block that reads the old state is the one
    // that writes the new one, each thread its own elements, so that no block reads a state that is already new.
    int first = 0, other = -1;
    float* st = nullptr;
    if (mix) {
        const int b = PLM_SEQ_NO(tok_seq[t]);
        first = t == seq_start[b];
        other = first ? seq_start[b + 1] - 1 : t - 1;
        if (other == t) other = -1;
        st = state + (long)seq_slot[b] * state_stride;
    }
    const float* xr = x + (size_t)t * d;
    const float* xo = x + (size_t)(other < 0 ? t : other) * d;
    const float r = 1.0f / sqrtf(block_sum<NT>(row_sum_squares<NT>(xr, d), red) / (float)d + eps);
    float ro = r;
    if (other >= 0) ro = 1.0f / sqrtf(block_sum<NT>(row_sum_squares<NT>(xo, d), red) / (float)d + eps);
    for (int i = threadIdx.x; i < d; i += NT) {
        const float v = xr[i];
        const float a = v * r * w_a[i];
        float o = a;
        if (mix) {
            const float prev = first ? st[i] : xo[i] * ro * w_a[i];
            o = a + (prev - a) * mix[i];
            if (first) st[i] = other < 0 ? a : xo[i] * ro * w_a[i];
        }
        out_a[(size_t)t * d + i] = from_f32<To>(o);
        if (out_b) out_b[(size_t)t * d + i] = from_f32<To>(v * r * w_b[i]);
    }
}

// The same with rows whose width is a multiple of 4 and at most 4 * VPT * NT: four elements at a time, both rows in
// registers between the sums of squares and the results (VPT float4 a thread and row), so that x is read once.
template <typename To, int NT, int VPT>
__global__ void __launch_bounds__(NT)
norm_pair_shift_vec_kernel(const float* __restrict__ x, const float* __restrict__ w_a, const float* __restrict__ w_b,
                           const float* __restrict__ mix, float* __restrict__ state, long state_stride,
                           const int* __restrict__ tok_seq, const int* __restrict__ seq_start, const int* __restrict__ seq_slot,
                           To* __restrict__ out_a, To* __restrict__ out_b, int d, float eps) {
    __shared__ float red[66];
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    int first = 0, other = -1;
    float* st = nullptr;
    if (mix) {
        const int b = PLM_SEQ_NO(tok_seq[t]);
        first = t == seq_start[b];
        other = first ? seq_start[b + 1] - 1 : t - 1;
        if (other == t) other = -1;
        st = state + (long)seq_slot[b] * state_stride;
    }
    const float* xr = x + (size_t)t * d;
    const float* xo = x + (size_t)(other < 0 ? t : other) * d;
    float4 v[VPT], u[VPT];
    float ss = 0.f, so = 0.f;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
        const int i = (threadIdx.x + k * NT) * 4;
        if (i < d) {
            v[k] = load4(xr + i);
            ss += v[k].x * v[k].x + v[k].y * v[k].y + v[k].z * v[k].z + v[k].w * v[k].w;
            if (other >= 0) {
                u[k] = load4(xo + i);
                so += u[k].x * u[k].x + u[k].y * u[k].y + u[k].z * u[k].z + u[k].w * u[k].w;
            }
        }
    }
    float r, ro;
    if (other >= 0) {
        const float2 sums = block_sum2<NT>(ss, so, red);
        r = 1.0f / sqrtf(sums.x / (float)d + eps);
        ro = 1.0f / sqrtf(sums.y / (float)d + eps);
    } else {
        r = ro = 1.0f / sqrtf(block_sum<NT>(ss, red) / (float)d + eps);
    }
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
        const int i = (threadIdx.x + k * NT) * 4;
        if (i >= d) continue;
        const float4 wa = load4(w_a + i);
        const float4 a = make_float4(v[k].x * r * wa.x, v[k].y * r * wa.y, v[k].z * r * wa.z, v[k].w * r * wa.w);
        float4 o = a;
        if (mix) {
            float4 kept = a;                       // the row that goes into the state: the sequence's last of the step
            if (other >= 0) kept = make_float4(u[k].x * ro * wa.x, u[k].y * ro * wa.y, u[k].z * ro * wa.z, u[k].w * ro * wa.w);
            const float4 prev = first ? load4(st + i) : kept;
            const float4 m = load4(mix + i);
            o = make_float4(a.x + (prev.x - a.x) * m.x, a.y + (prev.y - a.y) * m.y, a.z + (prev.z - a.z) * m.z, a.w + (prev.w - a.w) * m.w);
            if (first) store4(st + i, kept);
        }
        store4(out_a + (size_t)t * d + i, o);
        if (out_b) {
            const float4 wb = load4(w_b + i);
            store4(out_b + (size_t)t * d + i, make_float4(v[k].x * r * wb.x, v[k].y * r * wb.y, v[k].z * r * wb.z, v[k].w * r * wb.w));
        }
    }
}

template <typename To>
static int norm_pair_shift_launch(const float* x, const float* w_a, const float* w_b, const float* mix, float* state,
                                  long state_stride, const int* tok_seq, const int* seq_start, const int* seq_slot, void* out_a,
                                  void* out_b, int n_tokens, int d, float eps, cudaStream_t stream) {
    const bool aligned = (((uintptr_t)x | (uintptr_t)w_a | (uintptr_t)w_b | (uintptr_t)mix | (uintptr_t)state) & 15) == 0 &&
                         (((uintptr_t)out_a | (uintptr_t)out_b) & 7) == 0 && state_stride % 4 == 0;
    // (which kernel runs, and with it the order of the sums, depends on the row's width and on alignments that a model fixes)
    // few registers a thread (VPT) so that many blocks share an SM: what a block waits for is its rows' arrival
#define NPS_LAUNCH(NT_, VPT_)                                                                                           \
    return plm_status_of(launch_pdl(norm_pair_shift_vec_kernel<To, NT_, VPT_>, dim3(n_tokens), dim3(NT_), 0, stream, x, w_a,  \
                                    w_b, mix, state, state_stride, tok_seq, seq_start, seq_slot, (To*)out_a, (To*)out_b, d, eps))
    if (d % 4 == 0 && aligned) {
        if (d <= 4 * 256) NPS_LAUNCH(256, 1);
        if (d <= 8 * 256) NPS_LAUNCH(256, 2);
        if (d <= 8 * 512) NPS_LAUNCH(512, 2);
        if (d <= 8 * 1024) NPS_LAUNCH(1024, 2);
        if (d <= 16 * 1024) NPS_LAUNCH(1024, 4);
    }
#undef NPS_LAUNCH
    return plm_status_of(launch_pdl(norm_pair_shift_kernel<To, 256>, dim3(n_tokens), dim3(256), 0, stream, x, w_a, w_b, mix,
                                    state, state_stride, tok_seq, seq_start, seq_slot, (To*)out_a, (To*)out_b, d, eps));
}

extern "C" int plm_norm_pair_shift(const float* x, const float* w_a, const float* w_b, const float* mix, float* state,
                                   long state_stride, const int* tok_seq, const int* seq_start, const int* seq_slot, void* out_a,
                                   void* out_b, int out_dtype, int n_tokens, int d, float eps, cudaStream_t stream) {
    if (n_tokens <= 0) return PLM_OK;
    if (d <= 0 || (mix != nullptr && (state == nullptr || state_stride < d))) return PLM_ERR_SHAPE;
    if (out_dtype == PLM_F32)
        return norm_pair_shift_launch<float>(x, w_a, w_b, mix, state, state_stride, tok_seq, seq_start, seq_slot, out_a, out_b,
                                             n_tokens, d, eps, stream);
    if (out_dtype == PLM_BF16)
        return norm_pair_shift_launch<bf16>(x, w_a, w_b, mix, state, state_stride, tok_seq, seq_start, seq_slot, out_a, out_b,
                                            n_tokens, d, eps, stream);
    return PLM_ERR_DTYPE;
}
