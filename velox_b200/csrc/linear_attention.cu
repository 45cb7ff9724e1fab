// Linear attention with a per-head decay, as a recurrence over a state in float32:
//   S_p = decay_h * S_(p-1) + k_p v_p^T        S: [D, Dv] per head and request
//   o_p = S_p^T q_p
// q, k [H, D] and v [H, Dv] of every token are found at columns q_col, k_col, v_col of a
// packed projection x [tokens, ldx] (element type T) and optionally passed through silu
// in float32 on the way in.  The state lives in a slot per request, [slot, H, D, Dv], is
// read at the start of a request's tokens of this step and written back at their end;
// outputs are float32 [tokens, H * Dv].
//
// This kernel walks a request's tokens one after the other: it is the decode kernel, and
// the prompt kernel for portions too short to be worth cutting into chunks.  A block owns 32
// columns of one head's state of one request; a thread owns every fourth row of one
// column (D / 4 values in registers).  Tokens are staged 16 at a time in shared memory.
// Every sum runs in an order fixed by D alone, so a position's output is the same bits
// however its request's tokens were cut into steps.
#include "common.cuh"
#include "mma_helpers.cuh"

#define LA_COLS 32
#define LA_SLICES 4
#define LA_CHUNK 16

__device__ __forceinline__ float la_silu(float z) { return z / (1.f + expf(-z)); }
// The activated q, k, v are stored in the projections' element type: a bfloat16 engine rounds them
// (as the chunked kernel's input is rounded), the 32-bit engine does not.
__device__ __forceinline__ float la_store(float v, const float*) { return v; }
__device__ __forceinline__ float la_store(float v, const bf16*) { return __bfloat162float(__float2bfloat16_rn(v)); }

template <typename T, int DR>
__global__ void __launch_bounds__(LA_COLS * LA_SLICES)
linear_attention_recurrent_kernel(const T* __restrict__ x, int ldx, int q_col, int k_col, int v_col,
                                  const float* __restrict__ decay, float* __restrict__ state,
                                  const int* __restrict__ cu_seqlens, const int* __restrict__ state_slots,
                                  float* __restrict__ out, int H, int D, int Dv, int act) {
    extern __shared__ float smem[];
    float* q_s = smem;                       // [LA_CHUNK][D]
    float* k_s = q_s + LA_CHUNK * D;         // [LA_CHUNK][D]
    float* v_s = k_s + LA_CHUNK * D;         // [LA_CHUNK][LA_COLS]
    const int col0 = blockIdx.x * LA_COLS, h = blockIdx.y, seq = blockIdx.z;
    const int col = threadIdx.x / LA_SLICES, slice = threadIdx.x % LA_SLICES;
    const int c = col0 + col;
    const bool live = c < Dv;
    const float dec = decay[h];
    pdl_wait();
    pdl_trigger();
    const int t0 = cu_seqlens[seq], t1 = cu_seqlens[seq + 1];
    float* st = state + (((size_t)state_slots[seq] * H + h) * D) * Dv;
    float S[DR];
#pragma unroll
    for (int i = 0; i < DR; ++i) {
        const int d = slice + LA_SLICES * i;
        S[i] = (live && d < D) ? st[(size_t)d * Dv + c] : 0.f;
    }
    for (int tb = t0; tb < t1; tb += LA_CHUNK) {
        const int n = min(LA_CHUNK, t1 - tb);
        __syncthreads();
        for (int i = threadIdx.x; i < n * D; i += blockDim.x) {
            const int tt = i / D, d = i - tt * D;
            const T* row = x + (size_t)(tb + tt) * ldx + (size_t)h * D + d;
            const float qv = to_f32(row[q_col]), kv = to_f32(row[k_col]);
            q_s[i] = act ? la_store(la_silu(qv), x) : qv;
            k_s[i] = act ? la_store(la_silu(kv), x) : kv;
        }
        for (int i = threadIdx.x; i < n * LA_COLS; i += blockDim.x) {
            const int tt = i / LA_COLS, cc = i - tt * LA_COLS;
            float vv = 0.f;
            if (col0 + cc < Dv) {
                vv = to_f32(x[(size_t)(tb + tt) * ldx + v_col + (size_t)h * Dv + col0 + cc]);
                if (act) vv = la_store(la_silu(vv), x);
            }
            v_s[i] = vv;
        }
        __syncthreads();
        for (int tt = 0; tt < n; ++tt) {
            const float v = v_s[tt * LA_COLS + col];
            const float* kq = k_s + tt * D;
            const float* qq = q_s + tt * D;
            float o = 0.f;
#pragma unroll
            for (int i = 0; i < DR; ++i) {
                const int d = slice + LA_SLICES * i;
                if (d < D) {
                    S[i] = fmaf(dec, S[i], kq[d] * v);
                    o = fmaf(S[i], qq[d], o);
                }
            }
            o += __shfl_xor_sync(0xffffffffu, o, 1);
            o += __shfl_xor_sync(0xffffffffu, o, 2);
            if (slice == 0 && live) out[(size_t)(tb + tt) * H * Dv + (size_t)h * Dv + c] = o;
        }
    }
#pragma unroll
    for (int i = 0; i < DR; ++i) {
        const int d = slice + LA_SLICES * i;
        if (live && d < D) st[(size_t)d * Dv + c] = S[i];
    }
}

template <typename T>
static int launch_linear_attention_recurrent(const T* x, int ldx, int q_col, int k_col, int v_col, const float* decay,
                                             float* state, const int* cu_seqlens, const int* state_slots, float* out,
                                             int seqs, int H, int D, int Dv, int act, cudaStream_t stream) {
    dim3 grid((Dv + LA_COLS - 1) / LA_COLS, H, seqs);
    const size_t smem = sizeof(float) * LA_CHUNK * (2 * D + LA_COLS);
    const int dr = (D + LA_SLICES - 1) / LA_SLICES;
#define LA_GO(DR)                                                                                                  \
    VX_LAUNCH_K(VX_K_ATTENTION, (linear_attention_recurrent_kernel<T, DR>), grid, LA_COLS * LA_SLICES, smem, stream, x, \
                ldx, q_col, k_col, v_col, decay, state, cu_seqlens, state_slots, out, H, D, Dv, act)
    if (dr <= 8) LA_GO(8);
    else if (dr <= 16) LA_GO(16);
    else if (dr <= 32) LA_GO(32);
    else LA_GO(64);
#undef LA_GO
    VX_LAUNCH_CHECK();
    return VX_OK;
}

extern "C" int vx_linear_attention_recurrent(const void* x, int ldx, int q_col, int k_col, int v_col, const float* decay,
                                             float* state, const int* cu_seqlens, const int* state_slots, float* out,
                                             int seqs, int H, int D, int Dv, int act, int dtype, cudaStream_t stream) {
    if (seqs <= 0) return VX_OK;
    if (H <= 0 || D <= 0 || Dv <= 0 || D > 256 || q_col < 0 || k_col < 0 || v_col < 0) return VX_ERR_SHAPE;
    if (seqs > 65535 || H > 65535) return VX_ERR_LIMIT;
    if (dtype == VX_F32)
        return launch_linear_attention_recurrent<float>((const float*)x, ldx, q_col, k_col, v_col, decay, state, cu_seqlens,
                                                        state_slots, out, seqs, H, D, Dv, act, stream);
    if (dtype == VX_BF16)
        return launch_linear_attention_recurrent<bf16>((const bf16*)x, ldx, q_col, k_col, v_col, decay, state, cu_seqlens,
                                                       state_slots, out, seqs, H, D, Dv, act, stream);
    return VX_ERR_DTYPE;
}

// ---------------------------------------------------------------------------------------------
// The same recurrence for prompt portions, in chunks of 64 tokens on the tensor cores (bfloat16
// operands, float32 accumulators).  q, k, v here are the ACTIVATED projections, rounded to
// bfloat16 (the recurrent kernel rounds the same way when its input is bfloat16, so both kernels
// see the same numbers).  For a chunk of n tokens that follows the state S (i, j count from 0):
//   A[i, j] = q_i . k_j * decay^(i - j) for j <= i, else 0          scores, float32
//   o_i     = sum_j A[i, j] v_j + decay^(i + 1) * (q_i^T S)
//   S'      = decay^n S + sum_j k_j (decay^(n - 1 - j) v_j)^T
// Nothing is ever divided by a power of the decay.  What is not exactly a bfloat16 number goes into
// a product as two bfloat16 halves, hi + lo (16 bits of mantissa together): the masked scores A,
// the state S and the scaled values; q and k are exact.  The state itself stays in float32, in the
// accumulator registers of the product that updates it, from a request's first chunk of the step
// to its last.
//
// grid (tiles of DVT columns of the head's values, head, request); 4 warps.  Warp w owns rows
// 16 w .. of the chunk's outputs and a share of the state's rows.  Q, K, V tiles of the next
// chunk are fetched with cp.async while the current one is computed.
#define LC_CHUNK 64
#define LC_WARPS 4

template <int CH> __device__ __forceinline__ int lc_swz(int r, int cc) {
    return CH >= 8 ? (cc ^ (r & 7)) : (cc ^ ((r >> 1) & 3));
}

__device__ __forceinline__ void lc_split(float a, float b, unsigned& hi, unsigned& lo) {
    const __nv_bfloat162 h2 = __floats2bfloat162_rn(a, b);
    const float2 back = __bfloat1622float2(h2);
    hi = *reinterpret_cast<const unsigned*>(&h2);
    lo = pack_bf16(a - back.x, b - back.y);
}

template <int D, int DVT>
__global__ void __launch_bounds__(LC_WARPS * 32)
linear_attention_chunked_kernel(const bf16* __restrict__ x, int ldx, int q_col, int k_col, int v_col,
                                const float* __restrict__ decay, float* __restrict__ state,
                                const int* __restrict__ cu_seqlens, const int* __restrict__ state_slots,
                                float* __restrict__ out, int H, int Dv) {
    extern __shared__ __align__(128) unsigned char lc_smem[];
    constexpr int QCH = D / 8, VCH = DVT / 8;
    constexpr int QK_BYTES = LC_CHUNK * D * 2, V_BYTES = LC_CHUNK * DVT * 2, S_BYTES = D * DVT * 2;
    constexpr int STAGE = 2 * QK_BYTES + V_BYTES;
    constexpr int NM = D / 16;                        // 16-row tiles of the state
    constexpr int MT = NM >= 4 ? NM / 4 : 1;          // ... of which a warp owns MT
    constexpr int NSPLIT = NM >= 4 ? 1 : 4 / NM;      // (a small state: warps share a row tile and split its columns)
    constexpr int NT_S = (DVT / 8) / NSPLIT;          // 8-column tiles of the state a warp owns
    unsigned char* tiles = lc_smem;                   // 2 stages x (Q, K, V)
    unsigned char* vs_hi = lc_smem + 2 * STAGE;       // values times decay^(n-1-j), two halves
    unsigned char* vs_lo = vs_hi + V_BYTES;
    unsigned char* s_hi = vs_lo + V_BYTES;            // the state before the chunk, two halves, [D][DVT]
    unsigned char* s_lo = s_hi + S_BYTES;

    const int col0 = blockIdx.x * DVT, h = blockIdx.y, seq = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const float dec = decay[h];
    const float log2d = log2f(dec);
    pdl_wait();
    pdl_trigger();
    const int t0 = cu_seqlens[seq], t1 = cu_seqlens[seq + 1];
    if (t1 <= t0) return;
    float* st = state + (((size_t)state_slots[seq] * H + h) * D) * Dv + col0;

    const int m_base = NM >= 4 ? warp * MT : warp % NM;
    const int n_base = NM >= 4 ? 0 : (warp / NM) * NT_S;
    float S[MT][NT_S][4];
#pragma unroll
    for (int a = 0; a < MT; ++a)
#pragma unroll
        for (int b = 0; b < NT_S; ++b)
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int d = (m_base + a) * 16 + (lane >> 2) + 8 * half;
                const int c = (n_base + b) * 8 + 2 * (lane & 3);
                const float2 v2 = *reinterpret_cast<const float2*>(st + (size_t)d * Dv + c);
                S[a][b][2 * half] = v2.x;
                S[a][b][2 * half + 1] = v2.y;
            }

    auto issue = [&](int tb, int stage) {
        unsigned char* qs = tiles + stage * STAGE;
        unsigned char* ks = qs + QK_BYTES;
        unsigned char* vs = ks + QK_BYTES;
        const int n = min(LC_CHUNK, t1 - tb);
        for (int c = threadIdx.x; c < LC_CHUNK * QCH; c += LC_WARPS * 32) {
            const int r = c / QCH, cc = c % QCH;
            const int dst = r * (D * 2) + (lc_swz<QCH>(r, cc) << 4);
            if (r < n) {
                const bf16* row = x + (size_t)(tb + r) * ldx + (size_t)h * D + cc * 8;
                cp_async16(qs + dst, row + q_col);
                cp_async16(ks + dst, row + k_col);
            } else {
                *reinterpret_cast<uint4*>(qs + dst) = make_uint4(0, 0, 0, 0);
                *reinterpret_cast<uint4*>(ks + dst) = make_uint4(0, 0, 0, 0);
            }
        }
        for (int c = threadIdx.x; c < LC_CHUNK * VCH; c += LC_WARPS * 32) {
            const int r = c / VCH, cc = c % VCH;
            const int dst = r * (DVT * 2) + (lc_swz<VCH>(r, cc) << 4);
            if (r < n) cp_async16(vs + dst, x + (size_t)(tb + r) * ldx + v_col + (size_t)h * Dv + col0 + cc * 8);
            else *reinterpret_cast<uint4*>(vs + dst) = make_uint4(0, 0, 0, 0);
        }
    };
    issue(t0, 0);
    cp_async_commit();

    const int mi = lane >> 3;
    int it = 0;
    for (int tb = t0; tb < t1; tb += LC_CHUNK, ++it) {
        const int stage = it & 1;
        const int n = min(LC_CHUNK, t1 - tb);
        if (tb + LC_CHUNK < t1) issue(tb + LC_CHUNK, stage ^ 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const unsigned char* qs = tiles + stage * STAGE;
        const unsigned char* ks = qs + QK_BYTES;
        const unsigned char* vs = ks + QK_BYTES;
        // the state before the chunk, as two bfloat16 halves, for q^T S
#pragma unroll
        for (int a = 0; a < MT; ++a)
#pragma unroll
            for (int b = 0; b < NT_S; ++b)
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    const int d = (m_base + a) * 16 + (lane >> 2) + 8 * half;
                    const int c = (n_base + b) * 8 + 2 * (lane & 3);
                    unsigned hi, lo;
                    lc_split(S[a][b][2 * half], S[a][b][2 * half + 1], hi, lo);
                    const int at = d * (DVT * 2) + (lc_swz<VCH>(d, c >> 3) << 4) + (c & 7) * 2;
                    *reinterpret_cast<unsigned*>(s_hi + at) = hi;
                    *reinterpret_cast<unsigned*>(s_lo + at) = lo;
                }
        // the values times decay^(n - 1 - j), as two halves, for the state's update
        for (int c = threadIdx.x; c < LC_CHUNK * VCH; c += LC_WARPS * 32) {
            const int r = c / VCH, cc = c % VCH;
            const int at = r * (DVT * 2) + (lc_swz<VCH>(r, cc) << 4);
            const uint4 raw = *reinterpret_cast<const uint4*>(vs + at);
            const __nv_bfloat162* v2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
            const float f = r < n ? exp2f((float)(n - 1 - r) * log2d) : 0.f;
            uint4 hi, lo;
            unsigned* hp = reinterpret_cast<unsigned*>(&hi);
            unsigned* lp = reinterpret_cast<unsigned*>(&lo);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 v = __bfloat1622float2(v2[e]);
                lc_split(v.x * f, v.y * f, hp[e], lp[e]);
            }
            *reinterpret_cast<uint4*>(vs_hi + at) = hi;
            *reinterpret_cast<uint4*>(vs_lo + at) = lo;
        }
        __syncthreads();

        // ---- the chunk's outputs: rows 16 warp .. of this warp ----
        if (warp * 16 < n) {
            unsigned qf[D / 16][4];
            {
                const int r = warp * 16 + ((mi & 1) << 3) + (lane & 7);
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const int cc = 2 * kk + (mi >> 1);
                    ldmatrix_x4(qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3], qs + r * (D * 2) + (lc_swz<QCH>(r, cc) << 4));
                }
            }
            float o[DVT / 8][4], oi[DVT / 8][4];
#pragma unroll
            for (int i = 0; i < DVT / 8; ++i)
#pragma unroll
                for (int c = 0; c < 4; ++c) o[i][c] = oi[i][c] = 0.f;
            // q^T S (both halves of S)
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
                const int r = kk * 16 + ((mi & 1) << 3) + (lane & 7);
#pragma unroll
                for (int nt = 0; nt < DVT / 8; nt += 2) {
                    const int at = r * (DVT * 2) + (lc_swz<VCH>(r, nt + (mi >> 1)) << 4);
                    unsigned b00, b01, b10, b11;
                    ldmatrix_x4_trans(b00, b01, b10, b11, s_hi + at);
                    mma_bf16(oi[nt], qf[kk], b00, b01);
                    mma_bf16(oi[nt + 1], qf[kk], b10, b11);
                    ldmatrix_x4_trans(b00, b01, b10, b11, s_lo + at);
                    mma_bf16(oi[nt], qf[kk], b00, b01);
                    mma_bf16(oi[nt + 1], qf[kk], b10, b11);
                }
            }
            const int i0 = warp * 16 + (lane >> 2), i1 = i0 + 8;   // the two rows this thread holds
            {
                const float f0 = exp2f((float)(i0 + 1) * log2d), f1 = exp2f((float)(i1 + 1) * log2d);
#pragma unroll
                for (int nt = 0; nt < DVT / 8; ++nt) {
                    o[nt][0] = oi[nt][0] * f0; o[nt][1] = oi[nt][1] * f0;
                    o[nt][2] = oi[nt][2] * f1; o[nt][3] = oi[nt][3] * f1;
                }
            }
            // scores of the chunk, 16 keys at a time, only up to the warp's diagonal
            const int rr = ((mi >> 1) << 3) + (lane & 7);
#pragma unroll
            for (int kg = 0; kg < LC_CHUNK / 16; ++kg) {
                if (kg * 16 > warp * 16 + 15) continue;   // (warp-uniform: every key of the group lies after the warp's rows)
                float sc[2][4];
#pragma unroll
                for (int c = 0; c < 4; ++c) sc[0][c] = sc[1][c] = 0.f;
                const int r = kg * 16 + rr;
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const int cc = 2 * kk + (mi & 1);
                    unsigned b00, b01, b10, b11;
                    ldmatrix_x4(b00, b01, b10, b11, ks + r * (D * 2) + (lc_swz<QCH>(r, cc) << 4));
                    mma_bf16(sc[0], qf[kk], b00, b01);
                    mma_bf16(sc[1], qf[kk], b10, b11);
                }
#pragma unroll
                for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const int j = kg * 16 + nt * 8 + ((lane & 3) << 1) + (c & 1);
                        const int i = (c & 2) ? i1 : i0;
                        sc[nt][c] = j <= i ? sc[nt][c] * exp2f((float)(i - j) * log2d) : 0.f;
                    }
                unsigned hi[4], lw[4];
                lc_split(sc[0][0], sc[0][1], hi[0], lw[0]);
                lc_split(sc[0][2], sc[0][3], hi[1], lw[1]);
                lc_split(sc[1][0], sc[1][1], hi[2], lw[2]);
                lc_split(sc[1][2], sc[1][3], hi[3], lw[3]);
                const int rv = kg * 16 + ((mi & 1) << 3) + (lane & 7);
#pragma unroll
                for (int nt = 0; nt < DVT / 8; nt += 2) {
                    unsigned v00, v01, v10, v11;
                    ldmatrix_x4_trans(v00, v01, v10, v11, vs + rv * (DVT * 2) + (lc_swz<VCH>(rv, nt + (mi >> 1)) << 4));
                    mma_bf16(o[nt], hi, v00, v01);
                    mma_bf16(o[nt + 1], hi, v10, v11);
                    mma_bf16(o[nt], lw, v00, v01);
                    mma_bf16(o[nt + 1], lw, v10, v11);
                }
            }
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int i = half ? i1 : i0;
                if (i >= n) continue;
                float* dst = out + (size_t)(tb + i) * H * Dv + (size_t)h * Dv + col0 + 2 * (lane & 3);
#pragma unroll
                for (int nt = 0; nt < DVT / 8; ++nt)
                    *reinterpret_cast<float2*>(dst + nt * 8) = make_float2(o[nt][2 * half], o[nt][2 * half + 1]);
            }
        }

        // ---- the state after the chunk: S = decay^n S + K^T (values scaled) ----
        {
            const float fn = exp2f((float)n * log2d);
#pragma unroll
            for (int a = 0; a < MT; ++a)
#pragma unroll
                for (int b = 0; b < NT_S; ++b)
#pragma unroll
                    for (int c = 0; c < 4; ++c) S[a][b][c] *= fn;
#pragma unroll
            for (int kk = 0; kk < LC_CHUNK / 16; ++kk) {
                if (kk * 16 >= n) continue;   // (uniform: tokens past the chunk's end are zero)
                const int rv = kk * 16 + ((mi & 1) << 3) + (lane & 7);
#pragma unroll
                for (int a = 0; a < MT; ++a) {
                    // A = K^T: rows d of tile m_base + a, columns the 16 tokens of step kk; transposed load from K [token][d]
                    unsigned kf[4];
                    const int rk = kk * 16 + ((mi >> 1) << 3) + (lane & 7);
                    const int cc = 2 * (m_base + a) + (mi & 1);
                    ldmatrix_x4_trans(kf[0], kf[1], kf[2], kf[3], ks + rk * (D * 2) + (lc_swz<QCH>(rk, cc) << 4));
#pragma unroll
                    for (int b = 0; b < NT_S; b += 2) {
                        const int at = rv * (DVT * 2) + (lc_swz<VCH>(rv, n_base + b + (mi >> 1)) << 4);
                        unsigned v00, v01, v10, v11;
                        ldmatrix_x4_trans(v00, v01, v10, v11, vs_hi + at);
                        mma_bf16(S[a][b], kf, v00, v01);
                        mma_bf16(S[a][b + 1], kf, v10, v11);
                        ldmatrix_x4_trans(v00, v01, v10, v11, vs_lo + at);
                        mma_bf16(S[a][b], kf, v00, v01);
                        mma_bf16(S[a][b + 1], kf, v10, v11);
                    }
                }
            }
        }
        __syncthreads();   // every warp is done with this stage and the halves before they are written again
    }
    cp_async_wait<0>();
#pragma unroll
    for (int a = 0; a < MT; ++a)
#pragma unroll
        for (int b = 0; b < NT_S; ++b)
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int d = (m_base + a) * 16 + (lane >> 2) + 8 * half;
                const int c = (n_base + b) * 8 + 2 * (lane & 3);
                *reinterpret_cast<float2*>(st + (size_t)d * Dv + c) = make_float2(S[a][b][2 * half], S[a][b][2 * half + 1]);
            }
}

template <int D, int DVT>
static int launch_linear_attention_chunked(const bf16* x, int ldx, int q_col, int k_col, int v_col, const float* decay,
                                           float* state, const int* cu_seqlens, const int* state_slots, float* out,
                                           int seqs, int H, int Dv, cudaStream_t stream) {
    const size_t smem = 2 * (2 * (size_t)LC_CHUNK * D * 2 + (size_t)LC_CHUNK * DVT * 2) + 2 * (size_t)LC_CHUNK * DVT * 2 +
                        2 * (size_t)D * DVT * 2;
    static bool configured[VX_MAX_DEVICES];
    if (int rc = vx_configure_smem(linear_attention_chunked_kernel<D, DVT>, smem, configured)) return rc;
    dim3 grid(Dv / DVT, H, seqs);
    VX_LAUNCH_K(VX_K_ATTENTION, (linear_attention_chunked_kernel<D, DVT>), grid, LC_WARPS * 32, smem, stream, x, ldx, q_col,
                k_col, v_col, decay, state, cu_seqlens, state_slots, out, H, Dv);
    VX_LAUNCH_CHECK();
    return VX_OK;
}

// x: bfloat16 rows with the ACTIVATED q, k [H, D] and v [H, Dv] at the given columns.  D 32, 64 or 128; Dv a
// multiple of 32; columns and row stride multiples of 8 elements.
extern "C" int vx_linear_attention_chunked(const void* x, int ldx, int q_col, int k_col, int v_col, const float* decay,
                                           float* state, const int* cu_seqlens, const int* state_slots, float* out,
                                           int seqs, int H, int D, int Dv, cudaStream_t stream) {
    if (seqs <= 0) return VX_OK;
    if (H <= 0 || Dv <= 0 || Dv % 32 || q_col < 0 || k_col < 0 || v_col < 0) return VX_ERR_SHAPE;
    if (seqs > 65535 || H > 65535) return VX_ERR_LIMIT;
    if ((ldx | q_col | k_col | v_col) & 7 || (((uintptr_t)x) & 15) || (((uintptr_t)out) & 7) || (((uintptr_t)state) & 7))
        return VX_ERR_ALIGN;
#define LC_GO(D_, V_)                                                                                                  \
    if (D == D_ && Dv % V_ == 0)                                                                                       \
        return launch_linear_attention_chunked<D_, V_>((const bf16*)x, ldx, q_col, k_col, v_col, decay, state, cu_seqlens, \
                                                       state_slots, out, seqs, H, Dv, stream)
    LC_GO(32, 64); LC_GO(32, 32); LC_GO(64, 64); LC_GO(64, 32); LC_GO(128, 64); LC_GO(128, 32);
#undef LC_GO
    return VX_ERR_SHAPE;
}

// ---------------------------------------------------------------------------------------------
// The same chunks worked on side by side, for steps whose portions are long: a request's chunks no
// longer wait for one another.
//   1. every chunk's own contribution U_c = sum_j k_j (decay^(n - 1 - j) v_j)^T, all chunks at once
//   2. per request and state element, chunk after chunk (a few multiply-adds each): the state before chunk c
//      is written where U_c was, then state = decay^n state + U_c; the last one goes back to the slot
//   3. every chunk's outputs from its scores and the state before it, all chunks at once
// Blocks find their chunk by walking the requests' lengths; the grid is sized for tokens / 64 + requests
// chunks and the blocks beyond the real number leave.  The sums are the sequential kernel's.
struct LcChunk { int seq, first, n, index; };   // request, first token row, tokens, number among all chunks

__device__ __forceinline__ LcChunk lc_find_chunk(const int* __restrict__ cu_seqlens, int seqs, int c) {
    int base = 0;
    for (int s = 0; s < seqs; ++s) {
        const int t0 = cu_seqlens[s], len = cu_seqlens[s + 1] - t0;
        const int nc = (len + LC_CHUNK - 1) / LC_CHUNK;
        if (c < base + nc) return {s, t0 + (c - base) * LC_CHUNK, min(LC_CHUNK, len - (c - base) * LC_CHUNK), c};
        base += nc;
    }
    return {-1, 0, 0, c};
}

template <int D, int DVT, bool OUTPUTS>
__global__ void __launch_bounds__(LC_WARPS * 32)
linear_attention_chunk_kernel(const bf16* __restrict__ x, int ldx, int q_col, int k_col, int v_col,
                              const float* __restrict__ decay, float* __restrict__ scratch,
                              const int* __restrict__ cu_seqlens, int seqs, float* __restrict__ out, int H, int Dv) {
    extern __shared__ __align__(128) unsigned char lc_smem[];
    constexpr int QCH = D / 8, VCH = DVT / 8;
    constexpr int QK_BYTES = LC_CHUNK * D * 2, V_BYTES = LC_CHUNK * DVT * 2, S_BYTES = D * DVT * 2;
    constexpr int NM = D / 16;
    constexpr int MT = NM >= 4 ? NM / 4 : 1;
    constexpr int NSPLIT = NM >= 4 ? 1 : 4 / NM;
    constexpr int NT_S = (DVT / 8) / NSPLIT;
    unsigned char* qs = lc_smem;                  // (outputs only)
    unsigned char* ks = qs + QK_BYTES;
    unsigned char* vs = ks + QK_BYTES;
    unsigned char* b_hi = vs + V_BYTES;           // scaled values (state pass) or the state before the chunk (outputs)
    unsigned char* b_lo = b_hi + (OUTPUTS ? S_BYTES : V_BYTES);
    const int col0 = blockIdx.x * DVT, h = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, mi = lane >> 3;
    const float log2d = log2f(decay[h]);
    pdl_wait();
    pdl_trigger();
    const LcChunk ch = lc_find_chunk(cu_seqlens, seqs, blockIdx.z);
    if (ch.seq < 0) return;
    const int n = ch.n;
    float* mine = scratch + (((size_t)ch.index * H + h) * D) * Dv + col0;   // U_c, then the state before the chunk
    for (int c = threadIdx.x; c < LC_CHUNK * QCH; c += LC_WARPS * 32) {
        const int r = c / QCH, cc = c % QCH;
        const int dst = r * (D * 2) + (lc_swz<QCH>(r, cc) << 4);
        if (r < n) {
            const bf16* row = x + (size_t)(ch.first + r) * ldx + (size_t)h * D + cc * 8;
            if (OUTPUTS) cp_async16(qs + dst, row + q_col);
            cp_async16(ks + dst, row + k_col);
        } else {
            if (OUTPUTS) *reinterpret_cast<uint4*>(qs + dst) = make_uint4(0, 0, 0, 0);
            *reinterpret_cast<uint4*>(ks + dst) = make_uint4(0, 0, 0, 0);
        }
    }
    for (int c = threadIdx.x; c < LC_CHUNK * VCH; c += LC_WARPS * 32) {
        const int r = c / VCH, cc = c % VCH;
        const int dst = r * (DVT * 2) + (lc_swz<VCH>(r, cc) << 4);
        if (r < n) cp_async16(vs + dst, x + (size_t)(ch.first + r) * ldx + v_col + (size_t)h * Dv + col0 + cc * 8);
        else *reinterpret_cast<uint4*>(vs + dst) = make_uint4(0, 0, 0, 0);
    }
    cp_async_commit();
    if (OUTPUTS) {
        // the state before the chunk, float32 in the scratch, as two bfloat16 halves [D][DVT]
        for (int c = threadIdx.x; c < D * VCH; c += LC_WARPS * 32) {
            const int d = c / VCH, cc = c % VCH;
            const float4 a = *reinterpret_cast<const float4*>(mine + (size_t)d * Dv + cc * 8);
            const float4 b = *reinterpret_cast<const float4*>(mine + (size_t)d * Dv + cc * 8 + 4);
            uint4 hi, lo;
            lc_split(a.x, a.y, hi.x, lo.x); lc_split(a.z, a.w, hi.y, lo.y);
            lc_split(b.x, b.y, hi.z, lo.z); lc_split(b.z, b.w, hi.w, lo.w);
            const int at = d * (DVT * 2) + (lc_swz<VCH>(d, cc) << 4);
            *reinterpret_cast<uint4*>(b_hi + at) = hi;
            *reinterpret_cast<uint4*>(b_lo + at) = lo;
        }
    }
    cp_async_wait<0>();
    __syncthreads();
    if (!OUTPUTS) {
        for (int c = threadIdx.x; c < LC_CHUNK * VCH; c += LC_WARPS * 32) {
            const int r = c / VCH, cc = c % VCH;
            const int at = r * (DVT * 2) + (lc_swz<VCH>(r, cc) << 4);
            const uint4 raw = *reinterpret_cast<const uint4*>(vs + at);
            const __nv_bfloat162* v2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
            const float f = r < n ? exp2f((float)(n - 1 - r) * log2d) : 0.f;
            uint4 hi, lo;
            unsigned* hp = reinterpret_cast<unsigned*>(&hi);
            unsigned* lp = reinterpret_cast<unsigned*>(&lo);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 v = __bfloat1622float2(v2[e]);
                lc_split(v.x * f, v.y * f, hp[e], lp[e]);
            }
            *reinterpret_cast<uint4*>(b_hi + at) = hi;
            *reinterpret_cast<uint4*>(b_lo + at) = lo;
        }
        __syncthreads();
        const int m_base = NM >= 4 ? warp * MT : warp % NM;
        const int n_base = NM >= 4 ? 0 : (warp / NM) * NT_S;
        float S[MT][NT_S][4];
#pragma unroll
        for (int a = 0; a < MT; ++a)
#pragma unroll
            for (int b = 0; b < NT_S; ++b)
#pragma unroll
                for (int c = 0; c < 4; ++c) S[a][b][c] = 0.f;
#pragma unroll
        for (int kk = 0; kk < LC_CHUNK / 16; ++kk) {
            if (kk * 16 >= n) continue;
            const int rv = kk * 16 + ((mi & 1) << 3) + (lane & 7);
#pragma unroll
            for (int a = 0; a < MT; ++a) {
                unsigned kf[4];
                const int rk = kk * 16 + ((mi >> 1) << 3) + (lane & 7);
                const int cc = 2 * (m_base + a) + (mi & 1);
                ldmatrix_x4_trans(kf[0], kf[1], kf[2], kf[3], ks + rk * (D * 2) + (lc_swz<QCH>(rk, cc) << 4));
#pragma unroll
                for (int b = 0; b < NT_S; b += 2) {
                    const int at = rv * (DVT * 2) + (lc_swz<VCH>(rv, n_base + b + (mi >> 1)) << 4);
                    unsigned v00, v01, v10, v11;
                    ldmatrix_x4_trans(v00, v01, v10, v11, b_hi + at);
                    mma_bf16(S[a][b], kf, v00, v01);
                    mma_bf16(S[a][b + 1], kf, v10, v11);
                    ldmatrix_x4_trans(v00, v01, v10, v11, b_lo + at);
                    mma_bf16(S[a][b], kf, v00, v01);
                    mma_bf16(S[a][b + 1], kf, v10, v11);
                }
            }
        }
#pragma unroll
        for (int a = 0; a < MT; ++a)
#pragma unroll
            for (int b = 0; b < NT_S; ++b)
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    const int d = (m_base + a) * 16 + (lane >> 2) + 8 * half;
                    const int c = (n_base + b) * 8 + 2 * (lane & 3);
                    *reinterpret_cast<float2*>(mine + (size_t)d * Dv + c) = make_float2(S[a][b][2 * half], S[a][b][2 * half + 1]);
                }
        return;
    }
    // ---- outputs of the chunk (as in the sequential kernel) ----
    if (warp * 16 >= n) return;
    unsigned qf[D / 16][4];
    {
        const int r = warp * 16 + ((mi & 1) << 3) + (lane & 7);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
            ldmatrix_x4(qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3], qs + r * (D * 2) + (lc_swz<QCH>(r, 2 * kk + (mi >> 1)) << 4));
    }
    float o[DVT / 8][4], oi[DVT / 8][4];
#pragma unroll
    for (int i = 0; i < DVT / 8; ++i)
#pragma unroll
        for (int c = 0; c < 4; ++c) o[i][c] = oi[i][c] = 0.f;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
        const int r = kk * 16 + ((mi & 1) << 3) + (lane & 7);
#pragma unroll
        for (int nt = 0; nt < DVT / 8; nt += 2) {
            const int at = r * (DVT * 2) + (lc_swz<VCH>(r, nt + (mi >> 1)) << 4);
            unsigned b00, b01, b10, b11;
            ldmatrix_x4_trans(b00, b01, b10, b11, b_hi + at);
            mma_bf16(oi[nt], qf[kk], b00, b01);
            mma_bf16(oi[nt + 1], qf[kk], b10, b11);
            ldmatrix_x4_trans(b00, b01, b10, b11, b_lo + at);
            mma_bf16(oi[nt], qf[kk], b00, b01);
            mma_bf16(oi[nt + 1], qf[kk], b10, b11);
        }
    }
    const int i0 = warp * 16 + (lane >> 2), i1 = i0 + 8;
    {
        const float f0 = exp2f((float)(i0 + 1) * log2d), f1 = exp2f((float)(i1 + 1) * log2d);
#pragma unroll
        for (int nt = 0; nt < DVT / 8; ++nt) {
            o[nt][0] = oi[nt][0] * f0; o[nt][1] = oi[nt][1] * f0;
            o[nt][2] = oi[nt][2] * f1; o[nt][3] = oi[nt][3] * f1;
        }
    }
    const int rr = ((mi >> 1) << 3) + (lane & 7);
#pragma unroll
    for (int kg = 0; kg < LC_CHUNK / 16; ++kg) {
        if (kg * 16 > warp * 16 + 15) continue;
        float sc[2][4];
#pragma unroll
        for (int c = 0; c < 4; ++c) sc[0][c] = sc[1][c] = 0.f;
        const int r = kg * 16 + rr;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
            unsigned b00, b01, b10, b11;
            ldmatrix_x4(b00, b01, b10, b11, ks + r * (D * 2) + (lc_swz<QCH>(r, 2 * kk + (mi & 1)) << 4));
            mma_bf16(sc[0], qf[kk], b00, b01);
            mma_bf16(sc[1], qf[kk], b10, b11);
        }
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int j = kg * 16 + nt * 8 + ((lane & 3) << 1) + (c & 1);
                const int i = (c & 2) ? i1 : i0;
                sc[nt][c] = j <= i ? sc[nt][c] * exp2f((float)(i - j) * log2d) : 0.f;
            }
        unsigned hi[4], lw[4];
        lc_split(sc[0][0], sc[0][1], hi[0], lw[0]);
        lc_split(sc[0][2], sc[0][3], hi[1], lw[1]);
        lc_split(sc[1][0], sc[1][1], hi[2], lw[2]);
        lc_split(sc[1][2], sc[1][3], hi[3], lw[3]);
        const int rv = kg * 16 + ((mi & 1) << 3) + (lane & 7);
#pragma unroll
        for (int nt = 0; nt < DVT / 8; nt += 2) {
            unsigned v00, v01, v10, v11;
            ldmatrix_x4_trans(v00, v01, v10, v11, vs + rv * (DVT * 2) + (lc_swz<VCH>(rv, nt + (mi >> 1)) << 4));
            mma_bf16(o[nt], hi, v00, v01);
            mma_bf16(o[nt + 1], hi, v10, v11);
            mma_bf16(o[nt], lw, v00, v01);
            mma_bf16(o[nt + 1], lw, v10, v11);
        }
    }
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int i = half ? i1 : i0;
        if (i >= n) continue;
        float* dst = out + (size_t)(ch.first + i) * H * Dv + (size_t)h * Dv + col0 + 2 * (lane & 3);
#pragma unroll
        for (int nt = 0; nt < DVT / 8; ++nt)
            *reinterpret_cast<float2*>(dst + nt * 8) = make_float2(o[nt][2 * half], o[nt][2 * half + 1]);
    }
}

// One thread per state element of one head of one request: the chunks' contributions in order.
__global__ void linear_attention_scan_kernel(const float* __restrict__ decay, float* __restrict__ state,
                                             float* __restrict__ scratch, const int* __restrict__ cu_seqlens,
                                             const int* __restrict__ state_slots, int H, int cells) {
    pdl_wait();
    pdl_trigger();
    const int e = blockIdx.x * blockDim.x + threadIdx.x, h = blockIdx.y, seq = blockIdx.z;
    if (e >= cells) return;
    int first = 0;
    for (int s = 0; s < seq; ++s) first += (cu_seqlens[s + 1] - cu_seqlens[s] + LC_CHUNK - 1) / LC_CHUNK;
    const int len = cu_seqlens[seq + 1] - cu_seqlens[seq];
    const float log2d = log2f(decay[h]);
    float* st = state + ((size_t)state_slots[seq] * H + h) * cells + e;
    float run = *st;
    const int nchunks = (len + LC_CHUNK - 1) / LC_CHUNK;
    const size_t stride = (size_t)H * cells;
    float* p0 = scratch + ((size_t)first * H + h) * cells + e;
    const float full = exp2f((float)LC_CHUNK * log2d);
    // eight chunks' contributions are asked for at once (read one by one, each costs a memory latency: 33 chunks
    // took 50 us), then the chain of multiply-adds runs over them
    for (int c0 = 0; c0 < nchunks; c0 += 8) {
        float u[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) u[j] = c0 + j < nchunks ? p0[(size_t)(c0 + j) * stride] : 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            if (c0 + j < nchunks) {
                p0[(size_t)(c0 + j) * stride] = run;
                const int n = min(LC_CHUNK, len - (c0 + j) * LC_CHUNK);
                run = fmaf(n == LC_CHUNK ? full : exp2f((float)n * log2d), run, u[j]);
            }
        }
    }
    *st = run;
}

template <int D, int DVT>
static int launch_linear_attention_parallel(const bf16* x, int ldx, int q_col, int k_col, int v_col, const float* decay,
                                            float* state, float* scratch, const int* cu_seqlens, const int* state_slots,
                                            float* out, int seqs, int max_chunks, int H, int Dv, cudaStream_t stream) {
    const size_t smem_state = (size_t)LC_CHUNK * D * 2 * 2 + 3 * (size_t)LC_CHUNK * DVT * 2;
    const size_t smem_out = (size_t)LC_CHUNK * D * 2 * 2 + (size_t)LC_CHUNK * DVT * 2 + 2 * (size_t)D * DVT * 2;
    static bool conf_a[VX_MAX_DEVICES], conf_c[VX_MAX_DEVICES];
    if (int rc = vx_configure_smem(linear_attention_chunk_kernel<D, DVT, false>, smem_state, conf_a)) return rc;
    if (int rc = vx_configure_smem(linear_attention_chunk_kernel<D, DVT, true>, smem_out, conf_c)) return rc;
    dim3 grid(Dv / DVT, H, max_chunks);
    VX_LAUNCH_K(VX_K_ATTENTION, (linear_attention_chunk_kernel<D, DVT, false>), grid, LC_WARPS * 32, smem_state, stream, x, ldx,
                q_col, k_col, v_col, decay, scratch, cu_seqlens, seqs, out, H, Dv);
    const int cells = D * Dv;
    VX_LAUNCH_K(VX_K_ATTENTION, linear_attention_scan_kernel, dim3((cells + 255) / 256, H, seqs), 256, 0, stream, decay, state,
                scratch, cu_seqlens, state_slots, H, cells);
    VX_LAUNCH_K(VX_K_ATTENTION, (linear_attention_chunk_kernel<D, DVT, true>), grid, LC_WARPS * 32, smem_out, stream, x, ldx,
                q_col, k_col, v_col, decay, scratch, cu_seqlens, seqs, out, H, Dv);
    VX_LAUNCH_CHECK();
    return VX_OK;
}

// As vx_linear_attention_chunked, with a float32 scratch of max_chunks * H * D * Dv elements, max_chunks at
// least the chunks of 64 tokens of all requests together.
extern "C" int vx_linear_attention_parallel(const void* x, int ldx, int q_col, int k_col, int v_col, const float* decay,
                                            float* state, float* scratch, const int* cu_seqlens, const int* state_slots,
                                            float* out, int seqs, int max_chunks, int H, int D, int Dv, cudaStream_t stream) {
    if (seqs <= 0 || max_chunks <= 0) return VX_OK;
    if (H <= 0 || Dv <= 0 || Dv % 32 || q_col < 0 || k_col < 0 || v_col < 0 || !scratch) return VX_ERR_SHAPE;
    if (seqs > 65535 || H > 65535 || max_chunks > 65535) return VX_ERR_LIMIT;
    if ((ldx | q_col | k_col | v_col) & 7 || (((uintptr_t)x) & 15) || (((uintptr_t)out) & 7) || (((uintptr_t)state) & 7) ||
        (((uintptr_t)scratch) & 15))
        return VX_ERR_ALIGN;
#define LP_GO(D_, V_)                                                                                                     \
    if (D == D_ && Dv % V_ == 0)                                                                                          \
        return launch_linear_attention_parallel<D_, V_>((const bf16*)x, ldx, q_col, k_col, v_col, decay, state, scratch, \
                                                        cu_seqlens, state_slots, out, seqs, max_chunks, H, Dv, stream)
    LP_GO(32, 64); LP_GO(32, 32); LP_GO(64, 64); LP_GO(64, 32); LP_GO(128, 64); LP_GO(128, 32);
#undef LP_GO
    return VX_ERR_SHAPE;
}
