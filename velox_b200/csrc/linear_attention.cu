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

#define LA_COLS 32
#define LA_SLICES 4
#define LA_CHUNK 16

__device__ __forceinline__ float la_silu(float z) { return z / (1.f + expf(-z)); }

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
            q_s[i] = act ? la_silu(qv) : qv;
            k_s[i] = act ? la_silu(kv) : kv;
        }
        for (int i = threadIdx.x; i < n * LA_COLS; i += blockDim.x) {
            const int tt = i / LA_COLS, cc = i - tt * LA_COLS;
            float vv = 0.f;
            if (col0 + cc < Dv) {
                vv = to_f32(x[(size_t)(tb + tt) * ldx + v_col + (size_t)h * Dv + col0 + cc]);
                if (act) vv = la_silu(vv);
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
