// Row kernels around sublayers that norm their OUTPUT as well as their input, and
// the input embedding with a table of token pairs.
//
//   pair embedding      x = table[id] + pair_table[hash(previous id, id)], float32
//   merge_norm_add_norm the residual update of a block with norms on both sides of a
//                       sublayer, for a sublayer of one or two branches, fused with the
//                       norm that feeds the next sublayer
//   act                 an activation, element by element
//   gated_rmsnorm       rmsnorm(o) * w * sigmoid(g): the output stage of a linear-attention mixer
//   kv_store            new keys and values of any two sizes into their pages
//
// All statistics, sums and the residual stream are float32; T is the element type of
// the activations that feed matrix products.
#include "common.cuh"

// One block per token row t of the step.  The token before a step's first token of a
// request is that request's `last_token` (kept per state slot); the block of a
// request's first row reads it and then stores the request's last token of this step,
// so no other block touches that entry.  Position 0 has no previous token and takes
// the pair table's row `buckets`.
template <typename T>
__global__ void embedding_pair_kernel(const int* __restrict__ ids, const int* __restrict__ positions,
                                      const int* __restrict__ seq_of_token, const int* __restrict__ cu_seqlens,
                                      const int* __restrict__ state_slots, int* __restrict__ last_token,
                                      const T* __restrict__ table, const T* __restrict__ pair_table,
                                      float* __restrict__ out, int hidden, int vocab, int buckets,
                                      long long mul_prev, long long mul_cur) {
    pdl_wait();
    pdl_trigger();
    const int t = blockIdx.x;
    const int id = ids[t];
    float* o = out + (size_t)t * hidden;
    const int seq = seq_of_token[t];
    const int first = cu_seqlens[seq];
    int prev = -1;
    if (positions[t] > 0) prev = (t > first) ? ids[t - 1] : last_token[state_slots[seq]];
    __syncthreads();   // every thread has read the slot before one of them writes it
    if (t == first && threadIdx.x == 0) last_token[state_slots[seq]] = ids[cu_seqlens[seq + 1] - 1];
    if (id < 0 || id >= vocab || (positions[t] > 0 && (prev < 0 || prev >= vocab))) {
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = __int_as_float(0x7fc00000);
        return;
    }
    const long long row = positions[t] > 0 ? ((long long)prev * mul_prev + (long long)id * mul_cur) % buckets : buckets;
    const T* a = table + (size_t)id * hidden;
    const T* b = pair_table + (size_t)row * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = to_f32(a[i]) + to_f32(b[i]);
}

extern "C" int vx_embedding_pair(const int* ids, const int* positions, const int* seq_of_token, const int* cu_seqlens,
                                 const int* state_slots, int* last_token, const void* table, const void* pair_table,
                                 float* out, int tokens, int hidden, int vocab, int buckets, long long mul_prev,
                                 long long mul_cur, int dtype, cudaStream_t stream) {
    if (tokens <= 0) return VX_OK;
    if (hidden <= 0 || vocab <= 0 || buckets <= 0 || mul_prev < 0 || mul_cur < 0) return VX_ERR_SHAPE;
    const int threads = hidden >= 1024 ? 256 : 128;
    if (dtype == VX_F32)
        VX_LAUNCH_K(VX_K_ELEMENTWISE, (embedding_pair_kernel<float>), tokens, threads, 0, stream, ids, positions, seq_of_token,
                    cu_seqlens, state_slots, last_token, (const float*)table, (const float*)pair_table, out, hidden, vocab,
                    buckets, mul_prev, mul_cur);
    else if (dtype == VX_BF16)
        VX_LAUNCH_K(VX_K_ELEMENTWISE, (embedding_pair_kernel<bf16>), tokens, threads, 0, stream, ids, positions, seq_of_token,
                    cu_seqlens, state_slots, last_token, (const bf16*)table, (const bf16*)pair_table, out, hidden, vocab,
                    buckets, mul_prev, mul_cur);
    else
        return VX_ERR_DTYPE;
    VX_LAUNCH_CHECK();
    return VX_OK;
}

// One block per row.  With rms(v) = v * rsqrt(mean(v^2) + eps):
//   u = y0                                   one branch, no norm of its own (w0 null)
//   u = c0 * rms(y0) * w0 + c1 * rms(y1) * w1     two branches, each normed over the row
//   r = residual + mult * rms(u) * w_post    stored back into residual
//   out = rms(r) * w_next                    if w_next is given
//   out = r rounded to T                     if `out` is given without w_next (a next sublayer that reads the stream itself)
// Without w_post (and without a residual) out = u: the merged branches alone.
// The row of u (then r) is kept in shared memory between the passes; every thread
// re-reads only what it wrote itself.
template <typename T>
__global__ void merge_norm_add_norm_kernel(float* __restrict__ residual, const T* __restrict__ y0,
                                           const float* __restrict__ w0, float c0, const T* __restrict__ y1,
                                           const float* __restrict__ w1, float c1, const float* __restrict__ w_post,
                                           float mult, const float* __restrict__ w_next, T* __restrict__ out,
                                           int width, float eps) {
    extern __shared__ float row[];
    __shared__ float scratch[32];
    pdl_wait();
    pdl_trigger();
    const size_t base = (size_t)blockIdx.x * width;
    const float inv = 1.f / (float)width;
    float su = 0.f;
    if (w0) {
        float s0 = 0.f, s1 = 0.f;
        for (int i = threadIdx.x; i < width; i += blockDim.x) {
            const float a = to_f32(y0[base + i]);
            s0 += a * a;
            if (y1) { const float b = to_f32(y1[base + i]); s1 += b * b; }
        }
        s0 = block_sum(s0, scratch);
        const float r0 = c0 * rsqrtf(s0 * inv + eps);
        float r1 = 0.f;
        if (y1) { s1 = block_sum(s1, scratch); r1 = c1 * rsqrtf(s1 * inv + eps); }
        for (int i = threadIdx.x; i < width; i += blockDim.x) {
            float u = to_f32(y0[base + i]) * r0 * w0[i];
            if (y1) u += to_f32(y1[base + i]) * r1 * w1[i];
            row[i] = u;
            su += u * u;
        }
    } else {
        for (int i = threadIdx.x; i < width; i += blockDim.x) {
            const float u = to_f32(y0[base + i]);
            row[i] = u;
            su += u * u;
        }
    }
    if (!w_post) {   // the merged branches themselves, no residual
        for (int i = threadIdx.x; i < width; i += blockDim.x) out[base + i] = from_f32<T>(row[i]);
        return;
    }
    su = block_sum(su, scratch);
    const float ru = mult * rsqrtf(su * inv + eps);
    float sr = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float r = residual[base + i] + row[i] * ru * w_post[i];
        residual[base + i] = r;
        row[i] = r;
        sr += r * r;
    }
    if (!w_next) {
        if (out)
            for (int i = threadIdx.x; i < width; i += blockDim.x) out[base + i] = from_f32<T>(row[i]);
        return;
    }
    sr = block_sum(sr, scratch);
    const float rr = rsqrtf(sr * inv + eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x) out[base + i] = from_f32<T>(row[i] * rr * w_next[i]);
}

// The same with 8 elements per thread and access and the row in registers (width a multiple of 8, at most
// 8 * 256 * 4, 16-byte aligned pointers).
#define MN_THREADS 256

__device__ __forceinline__ void mn_load8(const float* p, float (&v)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void mn_load8(const bf16* p, float (&v)[8]) {
    const uint4 r = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
}
__device__ __forceinline__ void mn_store8(float* p, const float (&v)[8]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
__device__ __forceinline__ void mn_store8(bf16* p, const float (&v)[8]) {
    uint4 r;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = r;
}

template <typename T, int ITER>
__global__ void __launch_bounds__(MN_THREADS)
merge_norm_add_norm_vec_kernel(float* __restrict__ residual, const T* __restrict__ y0, const float* __restrict__ w0,
                               float c0, const T* __restrict__ y1, const float* __restrict__ w1, float c1,
                               const float* __restrict__ w_post, float mult, const float* __restrict__ w_next,
                               T* __restrict__ out, int width, float eps) {
    __shared__ float scratch[32];
    const int chunks = width >> 3;
    const size_t base = (size_t)blockIdx.x * width;
    const float inv = 1.f / (float)width;
    // the residual is older than the branches (they were computed from it): it is asked for before the wait
    float r[ITER][8];
    if (w_post) {
#pragma unroll
        for (int i = 0; i < ITER; ++i) {
            const int c = threadIdx.x + i * MN_THREADS;
            if (c < chunks) mn_load8(residual + base + c * 8, r[i]);
        }
    }
    pdl_wait();
    pdl_trigger();
    float u[ITER][8];
    float s0 = 0.f, s1 = 0.f;
#pragma unroll
    for (int i = 0; i < ITER; ++i) {
        const int c = threadIdx.x + i * MN_THREADS;
        if (c < chunks) {
            mn_load8(y0 + base + c * 8, u[i]);
#pragma unroll
            for (int j = 0; j < 8; ++j) s0 += u[i][j] * u[i][j];
        }
    }
    float su = s0;
    if (w0) {
        s0 = block_sum(s0, scratch);
        const float r0 = c0 * rsqrtf(s0 * inv + eps);
        float b[ITER][8];
        if (y1) {
#pragma unroll
            for (int i = 0; i < ITER; ++i) {
                const int c = threadIdx.x + i * MN_THREADS;
                if (c < chunks) {
                    mn_load8(y1 + base + c * 8, b[i]);
#pragma unroll
                    for (int j = 0; j < 8; ++j) s1 += b[i][j] * b[i][j];
                }
            }
            s1 = block_sum(s1, scratch);
        }
        const float r1 = y1 ? c1 * rsqrtf(s1 * inv + eps) : 0.f;
        su = 0.f;
#pragma unroll
        for (int i = 0; i < ITER; ++i) {
            const int c = threadIdx.x + i * MN_THREADS;
            if (c < chunks) {
                float wa[8], wb[8];
                mn_load8(w0 + c * 8, wa);
                if (y1) mn_load8(w1 + c * 8, wb);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    float v = u[i][j] * r0 * wa[j];
                    if (y1) v += b[i][j] * r1 * wb[j];
                    u[i][j] = v;
                    su += v * v;
                }
            }
        }
    }
    if (!w_post) {
#pragma unroll
        for (int i = 0; i < ITER; ++i) {
            const int c = threadIdx.x + i * MN_THREADS;
            if (c < chunks) mn_store8(out + base + c * 8, u[i]);
        }
        return;
    }
    su = block_sum(su, scratch);
    const float ru = mult * rsqrtf(su * inv + eps);
    float sr = 0.f;
#pragma unroll
    for (int i = 0; i < ITER; ++i) {
        const int c = threadIdx.x + i * MN_THREADS;
        if (c < chunks) {
            float wp[8];
            mn_load8(w_post + c * 8, wp);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                r[i][j] += u[i][j] * ru * wp[j];
                sr += r[i][j] * r[i][j];
            }
            mn_store8(residual + base + c * 8, r[i]);
            if (out && !w_next) mn_store8(out + base + c * 8, r[i]);
        }
    }
    if (!w_next) return;
    sr = block_sum(sr, scratch);
    const float rr = rsqrtf(sr * inv + eps);
#pragma unroll
    for (int i = 0; i < ITER; ++i) {
        const int c = threadIdx.x + i * MN_THREADS;
        if (c < chunks) {
            float wn[8], y[8];
            mn_load8(w_next + c * 8, wn);
#pragma unroll
            for (int j = 0; j < 8; ++j) y[j] = r[i][j] * rr * wn[j];
            mn_store8(out + base + c * 8, y);
        }
    }
}

template <typename T>
static int launch_merge_norm(float* residual, const T* y0, const float* w0, float c0, const T* y1, const float* w1, float c1,
                             const float* w_post, float mult, const float* w_next, T* out, int rows, int width, float eps,
                             cudaStream_t stream) {
    const bool aligned = !((((uintptr_t)residual) | ((uintptr_t)y0) | ((uintptr_t)y1) | ((uintptr_t)w0) | ((uintptr_t)w1) |
                            ((uintptr_t)w_post) | ((uintptr_t)w_next) | ((uintptr_t)out)) & 15);
    if (width % 8 == 0 && aligned && width <= 8 * MN_THREADS * 4) {
        const int iter = (width / 8 + MN_THREADS - 1) / MN_THREADS;
#define MN_GO(I)                                                                                                      \
    VX_LAUNCH_K(VX_K_ELEMENTWISE, (merge_norm_add_norm_vec_kernel<T, I>), rows, MN_THREADS, 0, stream, residual, y0, w0, \
                c0, y1, w1, c1, w_post, mult, w_next, out, width, eps)
        if (iter <= 1) MN_GO(1);
        else if (iter == 2) MN_GO(2);
        else MN_GO(4);
#undef MN_GO
    } else {
        const int threads = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
        VX_LAUNCH_K(VX_K_ELEMENTWISE, (merge_norm_add_norm_kernel<T>), rows, threads, sizeof(float) * width, stream, residual,
                    y0, w0, c0, y1, w1, c1, w_post, mult, w_next, out, width, eps);
    }
    VX_LAUNCH_CHECK();
    return VX_OK;
}

extern "C" int vx_merge_norm_add_norm(float* residual, const void* y0, const float* w0, float c0, const void* y1,
                                      const float* w1, float c1, const float* w_post, float mult, const float* w_next,
                                      void* out, int rows, int width, float eps, int dtype, cudaStream_t stream) {
    if (rows <= 0) return VX_OK;
    if (width <= 0 || !y0 || (y1 && (!w0 || !w1)) || (w_next && !out)) return VX_ERR_SHAPE;
    if (w_post ? !residual : (!out || !w0)) return VX_ERR_SHAPE;
    if (width > 12288) return VX_ERR_LIMIT;   // (the row lives in shared memory)
    if (dtype == VX_F32)
        return launch_merge_norm<float>(residual, (const float*)y0, w0, c0, (const float*)y1, w1, c1, w_post, mult, w_next,
                                        (float*)out, rows, width, eps, stream);
    if (dtype == VX_BF16)
        return launch_merge_norm<bf16>(residual, (const bf16*)y0, w0, c0, (const bf16*)y1, w1, c1, w_post, mult, w_next,
                                       (bf16*)out, rows, width, eps, stream);
    return VX_ERR_DTYPE;
}

// out = act(x), element by element; x [rows, width] with a row stride, out contiguous.
template <typename TI, typename TO>
__global__ void act_kernel(const TI* __restrict__ x, int ldx, TO* __restrict__ out, long long total, int width, int act) {
    pdl_wait();
    pdl_trigger();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / width;
        const int c = (int)(i - r * width);
        out[i] = from_f32<TO>(activation(to_f32(x[r * ldx + c]), act));
    }
}

// The same, 8 elements a thread and access (width and row stride multiples of 8, 16-byte aligned pointers).
template <typename TI, typename TO>
__global__ void act_vec_kernel(const TI* __restrict__ x, int ldx, TO* __restrict__ out, long long chunks, int row_chunks,
                               int act) {
    pdl_wait();
    pdl_trigger();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < chunks; i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / row_chunks;
        const int c = (int)(i - r * row_chunks) * 8;
        float v[8];
        mn_load8(x + r * ldx + c, v);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = activation(v[j], act);
        mn_store8(out + i * 8, v);
    }
}

extern "C" int vx_act(const void* x, int ldx, void* out, int rows, int width, int act, int in_dtype, int out_dtype,
                      cudaStream_t stream) {
    if (rows <= 0 || width <= 0) return VX_OK;
    if (ldx < width || act < 0 || act > VX_ACT_IDENTITY) return VX_ERR_SHAPE;
    const long long total = (long long)rows * width;
    if (width % 8 == 0 && ldx % 8 == 0 && !((((uintptr_t)x) | ((uintptr_t)out)) & 15)) {
        const long long chunks = total / 8;
        long long vb = (chunks + 255) / 256;
        if (vb > 148 * 16) vb = 148 * 16;
        if (in_dtype == VX_F32 && out_dtype == VX_F32)
            VX_LAUNCH_K(VX_K_ELEMENTWISE, (act_vec_kernel<float, float>), (int)vb, 256, 0, stream, (const float*)x, ldx, (float*)out, chunks, width / 8, act);
        else if (in_dtype == VX_BF16 && out_dtype == VX_BF16)
            VX_LAUNCH_K(VX_K_ELEMENTWISE, (act_vec_kernel<bf16, bf16>), (int)vb, 256, 0, stream, (const bf16*)x, ldx, (bf16*)out, chunks, width / 8, act);
        else if (in_dtype == VX_F32 && out_dtype == VX_BF16)
            VX_LAUNCH_K(VX_K_ELEMENTWISE, (act_vec_kernel<float, bf16>), (int)vb, 256, 0, stream, (const float*)x, ldx, (bf16*)out, chunks, width / 8, act);
        else
            return VX_ERR_DTYPE;
        VX_LAUNCH_CHECK();
        return VX_OK;
    }
    long long blocks = (total + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (in_dtype == VX_F32 && out_dtype == VX_F32)
        VX_LAUNCH_K(VX_K_ELEMENTWISE, (act_kernel<float, float>), (int)blocks, 256, 0, stream, (const float*)x, ldx, (float*)out, total, width, act);
    else if (in_dtype == VX_BF16 && out_dtype == VX_BF16)
        VX_LAUNCH_K(VX_K_ELEMENTWISE, (act_kernel<bf16, bf16>), (int)blocks, 256, 0, stream, (const bf16*)x, ldx, (bf16*)out, total, width, act);
    else if (in_dtype == VX_F32 && out_dtype == VX_BF16)
        VX_LAUNCH_K(VX_K_ELEMENTWISE, (act_kernel<float, bf16>), (int)blocks, 256, 0, stream, (const float*)x, ldx, (bf16*)out, total, width, act);
    else
        return VX_ERR_DTYPE;
    VX_LAUNCH_CHECK();
    return VX_OK;
}

// out[r, :] = o[r, :] * rsqrt(mean(o[r, :]^2) + eps) * w * sigmoid(g[r, :]); o float32 and
// contiguous, g of element type T with a row stride (a slice of a packed projection).
template <typename T>
__global__ void gated_rmsnorm_kernel(const float* __restrict__ o, const T* __restrict__ g, int ldg,
                                     const float* __restrict__ w, T* __restrict__ out, int width, float eps) {
    __shared__ float scratch[32];
    pdl_wait();
    pdl_trigger();
    const size_t base = (size_t)blockIdx.x * width;
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) { const float v = o[base + i]; ss += v * v; }
    ss = block_sum(ss, scratch);
    const float rstd = rsqrtf(ss / (float)width + eps);
    const T* gr = g + (size_t)blockIdx.x * ldg;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float z = to_f32(gr[i]);
        out[base + i] = from_f32<T>(o[base + i] * rstd * w[i] / (1.f + expf(-z)));
    }
}

extern "C" int vx_gated_rmsnorm(const float* o, const void* g, int ldg, const float* w, void* out, int rows, int width,
                                float eps, int dtype, cudaStream_t stream) {
    if (rows <= 0) return VX_OK;
    if (width <= 0 || ldg < width) return VX_ERR_SHAPE;
    const int threads = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
    if (dtype == VX_F32)
        VX_LAUNCH_K(VX_K_ELEMENTWISE, (gated_rmsnorm_kernel<float>), rows, threads, 0, stream, o, (const float*)g, ldg, w, (float*)out, width, eps);
    else if (dtype == VX_BF16)
        VX_LAUNCH_K(VX_K_ELEMENTWISE, (gated_rmsnorm_kernel<bf16>), rows, threads, 0, stream, o, (const bf16*)g, ldg, w, (bf16*)out, width, eps);
    else
        return VX_ERR_DTYPE;
    VX_LAUNCH_CHECK();
    return VX_OK;
}

// New keys [Hk, Dk] and values [Hk, Dv] of every token row, found at columns k_col and
// v_col of a packed projection, into the pools [page, Hk, S, Dk] and [page, Hk, S, Dv]
// at slot = page * S + offset (a negative slot writes nothing).
template <typename T>
__global__ void kv_store_kernel(const T* __restrict__ x, int ldx, int k_col, int v_col, const int* __restrict__ slot_mapping,
                                T* __restrict__ k_pool, T* __restrict__ v_pool, int Hk, int Dk, int Dv, int S) {
    pdl_wait();
    pdl_trigger();
    const int t = blockIdx.x;
    const int slot = slot_mapping[t];
    if (slot < 0) return;
    const int page = slot / S, off = slot % S;
    const T* row = x + (size_t)t * ldx;
    for (int i = threadIdx.x; i < Hk * Dk; i += blockDim.x) {
        const int h = i / Dk, d = i - h * Dk;
        k_pool[(((size_t)page * Hk + h) * S + off) * Dk + d] = row[k_col + i];
    }
    for (int i = threadIdx.x; i < Hk * Dv; i += blockDim.x) {
        const int h = i / Dv, d = i - h * Dv;
        v_pool[(((size_t)page * Hk + h) * S + off) * Dv + d] = row[v_col + i];
    }
}

extern "C" int vx_kv_store(const void* x, int ldx, int k_col, int v_col, const int* slot_mapping, void* k_pool,
                           void* v_pool, int tokens, int Hk, int Dk, int Dv, int S, int dtype, cudaStream_t stream) {
    if (tokens <= 0) return VX_OK;
    if (Hk <= 0 || Dk <= 0 || Dv <= 0 || S <= 0 || k_col < 0 || v_col < 0) return VX_ERR_SHAPE;
    if (dtype == VX_F32)
        VX_LAUNCH_K(VX_K_ROPE, (kv_store_kernel<float>), tokens, 128, 0, stream, (const float*)x, ldx, k_col, v_col, slot_mapping,
                    (float*)k_pool, (float*)v_pool, Hk, Dk, Dv, S);
    else if (dtype == VX_BF16)
        VX_LAUNCH_K(VX_K_ROPE, (kv_store_kernel<bf16>), tokens, 128, 0, stream, (const bf16*)x, ldx, k_col, v_col, slot_mapping,
                    (bf16*)k_pool, (bf16*)v_pool, Hk, Dk, Dv, S);
    else
        return VX_ERR_DTYPE;
    VX_LAUNCH_CHECK();
    return VX_OK;
}
