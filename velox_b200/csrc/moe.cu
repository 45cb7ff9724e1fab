// A routed feed-forward (mixture of experts) without a trip to the host:
//
//   route     per token: logits = W_r h + b in float32, the `top` largest (lowest index first
//             among equals), softmax over the chosen logits only; counts the tokens of every expert.
//             Or (mode 1) scores s = softmax(logits) over ALL outputs, choice by s + correction among the
//             outputs of the best `keep_groups` of `groups` equal groups of neighbours (a group's score:
//             its largest choice score), weights s * route_scale, not renormalised.  The router's last
//             outputs may be identity experts (no matrices: the token itself), and one more row of the
//             router's matrix may hold the gate of a shared expert, sigmoid(w . h) per token
//   plan      one block: where each expert's rows start in expert order, the list of row tiles
//             (expert, first row, rows) that the grouped products walk, and for every
//             assignment (token, k) its row in expert order
//   grouped product   C[p, :] = A[src(p), :] W_e^T for the rows p of each tile, W = [experts, N, K];
//             optionally with act(gate) * up on the accumulators (W's rows in tiles of 8 gate rows
//             followed by their 8 up rows)
//   combine   out[t] = sum_k weight[t, k] * y[row of (t, k)] (+ gate[t] * shared[t]) in float32, k ascending;
//             an assignment to an identity expert adds weight * h[t] instead
//
// The grid of a grouped product is sized for the worst case (assignments / tile rows + experts
// tiles); blocks beyond the step's real number of tiles leave at once.  Which tile a row falls
// into depends on the batch, but a row's sums run over k in ascending order whatever its tile, so
// a token's result does not depend on what else is in the step.
#include "mma_helpers.cuh"

#define MOE_MAX_EXPERTS 256
#define MOE_MAX_TOP 32

__device__ __forceinline__ void route_load8(const float* p, float (&v)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void route_load8(const bf16* p, float (&v)[8]) {
    const uint4 r = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h2[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
}

// Four consecutive elements of a token's row as they are loaded (one register pair or quad), and as floats.
template <typename T> struct RouteRow;
template <> struct RouteRow<float> {
    typedef float4 packed;
    static __device__ __forceinline__ void unpack(const float4& a, float (&v)[4]) { v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; }
};
template <> struct RouteRow<bf16> {
    typedef uint2 packed;
    static __device__ __forceinline__ void unpack(const uint2& r, float (&v)[4]) {
        const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&r);
        const float2 f0 = __bfloat1622float2(h2[0]), f1 = __bfloat1622float2(h2[1]);
        v[0] = f0.x; v[1] = f0.y; v[2] = f1.x; v[3] = f1.y;
    }
};

// What follows a token's logits z[0 .. E) (and z[E], the shared gate's, if there is one), by the token's warp: the
// shared gate, the scores, the choice and the weights, the experts' counters.  z, sc, gs (floats) and kept hold
// MOE_MAX_EXPERTS (+ 8) entries of this warp's own, zc and pick MOE_MAX_TOP.
__device__ __forceinline__ void route_select(float* z, float* sc, float* gs, unsigned char* kept, float* zc, int* pick, int lane, int t,
                                             int E, int top, int* __restrict__ chosen, float* __restrict__ weight,
                                             int* __restrict__ counts, int* __restrict__ pos, int mode,
                                             const float* __restrict__ correction, int groups, int keep_groups,
                                             float route_scale, float* __restrict__ shared_gate) {
    if (shared_gate && lane == 0) shared_gate[t] = 1.f / (1.f + expf(-z[E]));
    if (mode == 1) {
        float mx = -INFINITY;
        for (int e = lane; e < E; e += 32) mx = fmaxf(mx, z[e]);
        mx = warp_max(mx);
        float sum = 0.f;
        for (int e = lane; e < E; e += 32) { const float p = expf(z[e] - mx); sc[e] = p; sum += p; }
        sum = warp_sum(sum);
        for (int e = lane; e < E; e += 32) {
            const float v = sc[e] / sum;
            sc[e] = v;
            z[e] = v + (correction ? correction[e] : 0.f);   // the choice score; the weight stays v
        }
        __syncwarp();
        if (groups > 1 && keep_groups < groups) {
            const int gsize = E / groups;
            for (int g = lane; g < groups; g += 32) {
                float b = -INFINITY;
                for (int e = g * gsize; e < (g + 1) * gsize; ++e) b = fmaxf(b, z[e]);
                gs[g] = b;
                kept[g] = 0;
            }
            __syncwarp();
            for (int i = 0; i < keep_groups; ++i) {
                float best = -INFINITY;
                int arg = 0x7fffffff;
                for (int g = lane; g < groups; g += 32) {
                    const float v = gs[g];
                    if (!kept[g] && (v > best || (v == best && g < arg))) { best = v; arg = g; }
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) {
                    const float ob = __shfl_xor_sync(0xffffffffu, best, o);
                    const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
                    if (oa != 0x7fffffff && (arg == 0x7fffffff || ob > best || (ob == best && oa < arg))) { best = ob; arg = oa; }
                }
                if (lane == 0 && arg != 0x7fffffff) kept[arg] = 1;
                __syncwarp();
            }
            for (int e = lane; e < E; e += 32)
                if (!kept[e / gsize]) z[e] = -INFINITY;   // (not 0: a choice score may be negative)
            __syncwarp();
        }
    }
    for (int i = 0; i < top; ++i) {
        float best = -INFINITY;
        int arg = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float v = z[e];
            if (v > best || (v == best && e < arg)) { best = v; arg = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
            if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
        }
        if (lane == 0) {
            zc[i] = mode == 1 ? sc[arg] : best;
            z[arg] = -INFINITY;
            pick[i] = arg;
        }
        __syncwarp();
    }
    // a lane a choice: the experts' counters are asked all at once (one after the other each costs a trip to the L2)
    if (lane < top) {
        const int e = pick[lane];
        chosen[(size_t)t * top + lane] = e;
        float w;
        if (mode == 1) {
            w = zc[lane] * route_scale;
        } else {
            const float m = zc[0];
            float sum = 0.f;
            for (int i = 0; i < top; ++i) sum += expf(zc[i] - m);
            w = expf(zc[lane] - m) / sum;
        }
        weight[(size_t)t * top + lane] = w;
        pos[(size_t)t * top + lane] = atomicAdd(&counts[e], 1);
    }
}

#define ROUTE_KC 512
// `vec`: K a multiple of 8 and 16-byte aligned rows (the host checks); else element by element.
template <typename T>
__global__ void __launch_bounds__(128)
moe_route_kernel(const T* __restrict__ h, int ldh, const float* __restrict__ w_router, const float* __restrict__ bias,
                 int tokens, int K, int E, int top, int* __restrict__ chosen, float* __restrict__ weight,
                 int* __restrict__ counts, int* __restrict__ pos, int vec, int mode, const float* __restrict__ correction,
                 int groups, int keep_groups, float route_scale, float* __restrict__ shared_gate) {
    __shared__ float z_s[4][MOE_MAX_EXPERTS + 8];
    __shared__ float zc_s[4][MOE_MAX_TOP];
    __shared__ int pick_s[4][MOE_MAX_TOP];
    __shared__ float sc_s[4][MOE_MAX_EXPERTS];      // mode 1: the scores of all outputs
    __shared__ float gs_s[4][MOE_MAX_EXPERTS];      //         the groups' scores
    __shared__ unsigned char kept_s[4][MOE_MAX_EXPERTS];
    const int rows = E + (shared_gate ? 1 : 0);     // rows of the router's matrix: the outputs, then the shared gate's
    pdl_wait();
    pdl_trigger();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * 4 + warp;
    const bool valid = t < tokens;
    const T* row = h + (size_t)(valid ? t : 0) * ldh;
    float* z = z_s[warp];
    if (vec) {
        // Eight experts at a time, 512 k at a time: the block brings that piece of the router's matrix into shared
        // memory with every thread's loads in flight at once (read one after the other by a single warp they cost a
        // memory latency each: 25 us for 8 experts of 2,048), then each warp takes its token's 8 dot products from there.
        __shared__ __align__(16) float w_s[8][ROUTE_KC];
        for (int e0 = 0; e0 < rows; e0 += 8) {
            float acc[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] = 0.f;
            for (int k0 = 0; k0 < K; k0 += ROUTE_KC) {
                __syncthreads();
                float4 v[8];   // (a block of 128 threads: 8 loads each, all asked for before any is stored)
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const int idx = threadIdx.x + u * 128;
                    const int e = idx / (ROUTE_KC / 4), c = (idx % (ROUTE_KC / 4)) * 4;
                    v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (k0 + c < K) v[u] = *reinterpret_cast<const float4*>(w_router + (size_t)min(e0 + e, rows - 1) * K + k0 + c);
                }
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const int idx = threadIdx.x + u * 128;
                    *reinterpret_cast<float4*>(&w_s[idx / (ROUTE_KC / 4)][(idx % (ROUTE_KC / 4)) * 4]) = v[u];
                }
                __syncthreads();
                if (valid) {
                    for (int kk = lane * 8; kk < ROUTE_KC && k0 + kk < K; kk += 256) {
                        float hv[8];
                        route_load8(row + k0 + kk, hv);
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const float4 a = *reinterpret_cast<const float4*>(&w_s[j][kk]);
                            const float4 b = *reinterpret_cast<const float4*>(&w_s[j][kk + 4]);
                            acc[j] = fmaf(hv[0], a.x, acc[j]); acc[j] = fmaf(hv[1], a.y, acc[j]);
                            acc[j] = fmaf(hv[2], a.z, acc[j]); acc[j] = fmaf(hv[3], a.w, acc[j]);
                            acc[j] = fmaf(hv[4], b.x, acc[j]); acc[j] = fmaf(hv[5], b.y, acc[j]);
                            acc[j] = fmaf(hv[6], b.z, acc[j]); acc[j] = fmaf(hv[7], b.w, acc[j]);
                        }
                    }
                }
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float s = warp_sum(acc[j]);
                if (lane == 0 && e0 + j < rows) z[e0 + j] = s + ((bias && e0 + j < E) ? bias[e0 + j] : 0.f);
            }
        }
    } else if (valid) {
        for (int e = 0; e < rows; ++e) {
            const float* w = w_router + (size_t)e * K;
            float s = 0.f;
            for (int k = lane; k < K; k += 32) s = fmaf(to_f32(row[k]), w[k], s);
            s = warp_sum(s);
            if (lane == 0) z[e] = s + ((bias && e < E) ? bias[e] : 0.f);
        }
    }
    if (!valid) return;
    __syncwarp();
    route_select(z, sc_s[warp], gs_s[warp], kept_s[warp], zc_s[warp], pick_s[warp], lane, t, E, top, chosen, weight, counts, pos, mode,
                 correction, groups, keep_groups, route_scale, shared_gate);
}

// The same with the router's whole matrix resident in shared memory: a block brings it in once (before it waits for
// the step's earlier kernels: weights depend on none) and then walks its share of the tokens, 16 at a time, a warp a
// token.  A lane takes 4 consecutive k of every 128, so that a warp's reads of a row are one run of 512 bytes.  The
// warps' own arrays follow the matrix in the same dynamic shared memory, sized by the number of outputs.
#define ROUTE_R_WARPS 16
#define ROUTE_RESIDENT_MAX (220 * 1024)
// a warp's own arrays: four of `entries` floats (logits, scores, group scores, flags), the chosen scores and outputs
__host__ __device__ constexpr int route_warp_entries(int rows) { return ((rows + 7) & ~7) + 8; }
__host__ __device__ constexpr int route_warp_floats(int rows) { return 4 * route_warp_entries(rows) + 2 * MOE_MAX_TOP; }
template <typename T>
__global__ void __launch_bounds__(ROUTE_R_WARPS * 32)
moe_route_resident_kernel(const T* __restrict__ h, int ldh, const float* __restrict__ w_router, const float* __restrict__ bias,
                          int tokens, int K, int E, int top, int* __restrict__ chosen, float* __restrict__ weight,
                          int* __restrict__ counts, int* __restrict__ pos, int mode, const float* __restrict__ correction,
                          int groups, int keep_groups, float route_scale, float* __restrict__ shared_gate) {
    extern __shared__ __align__(16) float rw_s[];   // [rows][K], then per warp: z, scores, group scores, kept flags, chosen
    const int rows = E + (shared_gate ? 1 : 0);
    const int ep = route_warp_entries(rows);
    float* mine = rw_s + (size_t)rows * K + (size_t)(threadIdx.x >> 5) * route_warp_floats(rows);
    {
        const float4* src = reinterpret_cast<const float4*>(w_router);
        float4* dst = reinterpret_cast<float4*>(rw_s);
        const int n4 = rows * (K >> 2);
        int i = threadIdx.x;
        for (; i + 7 * ROUTE_R_WARPS * 32 < n4; i += 8 * ROUTE_R_WARPS * 32) {   // eight loads in flight a thread
            float4 v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) v[u] = src[i + u * ROUTE_R_WARPS * 32];
#pragma unroll
            for (int u = 0; u < 8; ++u) dst[i + u * ROUTE_R_WARPS * 32] = v[u];
        }
        for (; i < n4; i += ROUTE_R_WARPS * 32) dst[i] = src[i];
    }
    pdl_wait();
    pdl_trigger();
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float* z = mine;
    for (int t = blockIdx.x * ROUTE_R_WARPS + warp; t < tokens; t += gridDim.x * ROUTE_R_WARPS) {
        const T* row = h + (size_t)t * ldh;
        for (int e0 = 0; e0 < rows; e0 += 8) {
            float acc[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] = 0.f;
            // the token's row comes 2,048 (bfloat16) or 1,024 (float) k at a time, every load of such a piece asked for
            // before the first is used: one trip to memory a piece, not one every 128 k
            constexpr int PIECE = sizeof(T) == 2 ? 16 : 8;
            const int nr = min(8, rows - e0);
            for (int k0 = lane * 4; k0 < K; k0 += PIECE * 128) {
                typename RouteRow<T>::packed hp[PIECE];
#pragma unroll
                for (int c = 0; c < PIECE; ++c)
                    if (k0 + c * 128 < K) hp[c] = *reinterpret_cast<const typename RouteRow<T>::packed*>(row + k0 + c * 128);
#pragma unroll
                for (int c = 0; c < PIECE; ++c) {
                    const int k = k0 + c * 128;
                    if (k < K) {
                        float hv[4];
                        RouteRow<T>::unpack(hp[c], hv);
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            if (j < nr) {   // (the last group of rows may be short: nothing is read or added for the rest)
                                const float4 a = *reinterpret_cast<const float4*>(rw_s + (size_t)(e0 + j) * K + k);
                                acc[j] = fmaf(hv[0], a.x, acc[j]); acc[j] = fmaf(hv[1], a.y, acc[j]);
                                acc[j] = fmaf(hv[2], a.z, acc[j]); acc[j] = fmaf(hv[3], a.w, acc[j]);
                            }
                        }
                    }
                }
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float s = warp_sum(acc[j]);
                if (lane == 0 && e0 + j < rows) z[e0 + j] = s + ((bias && e0 + j < E) ? bias[e0 + j] : 0.f);
            }
        }
        __syncwarp();
        route_select(z, mine + ep, mine + 2 * ep, reinterpret_cast<unsigned char*>(mine + 3 * ep), mine + 4 * ep,
                     reinterpret_cast<int*>(mine + 4 * ep + MOE_MAX_TOP), lane, t, E, top,
                     chosen, weight, counts, pos, mode, correction, groups, keep_groups, route_scale, shared_gate);
        __syncwarp();
    }
}

// tiles: int3 per tile (expert, first row in expert order, rows); n_tiles[0] their number.
__global__ void __launch_bounds__(1024)
moe_plan_kernel(const int* __restrict__ chosen, const int* __restrict__ pos, int* __restrict__ counts, int assignments,
                int E, int tile_rows, int* __restrict__ offsets, int* __restrict__ tiles, int* __restrict__ n_tiles,
                int* __restrict__ src_of_row, int* __restrict__ row_of, int tile_experts) {
    __shared__ int off_s[MOE_MAX_EXPERTS + 1];
    __shared__ int cnt_s[MOE_MAX_EXPERTS];
    pdl_wait();
    pdl_trigger();
    for (int e = threadIdx.x; e < E; e += blockDim.x) cnt_s[e] = counts[e];   // (together: the walk below would wait for each)
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0, n = 0;
        for (int e = 0; e < E; ++e) {
            off_s[e] = run;
            offsets[e] = run;
            const int c = cnt_s[e];
            // (outputs from `tile_experts` on are identity experts: their rows keep a place, no product walks them)
            for (int r = 0; r < c && e < tile_experts; r += tile_rows) {
                tiles[3 * n] = e;
                tiles[3 * n + 1] = run + r;
                tiles[3 * n + 2] = min(tile_rows, c - r);
                ++n;
            }
            run += c;
        }
        off_s[E] = run;
        offsets[E] = run;
        n_tiles[0] = n;
    }
    __syncthreads();
    for (int a0 = threadIdx.x; a0 < assignments; a0 += 4 * blockDim.x) {   // (four assignments' loads in flight a thread)
        int c[4], q[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int a = a0 + u * blockDim.x;
            c[u] = a < assignments ? chosen[a] : 0;
            q[u] = a < assignments ? pos[a] : 0;
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int a = a0 + u * blockDim.x;
            if (a < assignments) {
                const int p = off_s[c[u]] + q[u];
                src_of_row[p] = a;
                row_of[a] = p;
            }
        }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x) counts[e] = 0;   // ready for the next step
}

// E: the router's outputs (experts, then `identity` identity experts).  mode 0: top-k of the logits, softmax over
// the chosen; mode 1: softmax over all, choice by score + correction within the best groups, weights score * route_scale.
// With `shared_gate` the router's matrix has one more row and shared_gate[t] = sigmoid(that row . h[t]).
extern "C" int vx_moe_route(const void* h, int ldh, const float* w_router, const float* bias, int tokens, int K, int E,
                            int top, int tile_rows, int* chosen, float* weight, int* counts, int* pos, int* offsets,
                            int* tiles, int* n_tiles, int* src_of_row, int* row_of, int dtype, int mode,
                            const float* correction, int groups, int keep_groups, float route_scale, int identity,
                            float* shared_gate, cudaStream_t stream) {
    if (tokens <= 0) return VX_OK;
    if (K <= 0 || E <= 0 || top <= 0 || top > E || tile_rows <= 0) return VX_ERR_SHAPE;
    if (mode < 0 || mode > 1 || identity < 0 || identity >= E) return VX_ERR_SHAPE;
    if (groups < 1) groups = 1;
    if (E % groups || keep_groups < 1 || keep_groups > groups || top > keep_groups * (E / groups)) return VX_ERR_SHAPE;
    if (E > MOE_MAX_EXPERTS || top > MOE_MAX_TOP) return VX_ERR_LIMIT;
    const int blocks = (tokens + 3) / 4;
    const int elt = dtype == VX_F32 ? 4 : 2;
    const int vec = K % 8 == 0 && (ldh * elt) % 16 == 0 && !(((uintptr_t)h) & 15) && !(((uintptr_t)w_router) & 15);
    // the router's matrix resident in shared memory where it fits (with the warps' own arrays behind it)
    const int mrows = E + (shared_gate ? 1 : 0);
    const size_t resident = ((size_t)mrows * K + (size_t)ROUTE_R_WARPS * route_warp_floats(mrows)) * sizeof(float);
    if (vec && resident <= ROUTE_RESIDENT_MAX && (dtype == VX_F32 || dtype == VX_BF16)) {
        static bool conf_f[VX_MAX_DEVICES], conf_b[VX_MAX_DEVICES];
        static int sms[VX_MAX_DEVICES];
        if (int rc = dtype == VX_F32 ? vx_configure_smem(moe_route_resident_kernel<float>, ROUTE_RESIDENT_MAX, conf_f)
                                     : vx_configure_smem(moe_route_resident_kernel<bf16>, ROUTE_RESIDENT_MAX, conf_b)) return rc;
        const int per_sm = 1;   // (512 threads with the token's row in registers: one block an SM)
        int rblocks = (tokens + ROUTE_R_WARPS - 1) / ROUTE_R_WARPS;
        if (rblocks > vx_sm_count(sms) * per_sm) rblocks = vx_sm_count(sms) * per_sm;
        if (dtype == VX_F32)
            VX_LAUNCH_K(VX_K_ELEMENTWISE, (moe_route_resident_kernel<float>), rblocks, ROUTE_R_WARPS * 32, resident, stream,
                        (const float*)h, ldh, w_router, bias, tokens, K, E, top, chosen, weight, counts, pos, mode, correction,
                        groups, keep_groups, route_scale, shared_gate);
        else
            VX_LAUNCH_K(VX_K_ELEMENTWISE, (moe_route_resident_kernel<bf16>), rblocks, ROUTE_R_WARPS * 32, resident, stream,
                        (const bf16*)h, ldh, w_router, bias, tokens, K, E, top, chosen, weight, counts, pos, mode, correction,
                        groups, keep_groups, route_scale, shared_gate);
    } else
    if (dtype == VX_F32)
        VX_LAUNCH_K(VX_K_ELEMENTWISE, (moe_route_kernel<float>), blocks, 128, 0, stream, (const float*)h, ldh, w_router, bias,
                    tokens, K, E, top, chosen, weight, counts, pos, vec, mode, correction, groups, keep_groups, route_scale,
                    shared_gate);
    else if (dtype == VX_BF16)
        VX_LAUNCH_K(VX_K_ELEMENTWISE, (moe_route_kernel<bf16>), blocks, 128, 0, stream, (const bf16*)h, ldh, w_router, bias,
                    tokens, K, E, top, chosen, weight, counts, pos, vec, mode, correction, groups, keep_groups, route_scale,
                    shared_gate);
    else
        return VX_ERR_DTYPE;
    VX_LAUNCH_K(VX_K_ELEMENTWISE, moe_plan_kernel, 1, 1024, 0, stream, (const int*)chosen, (const int*)pos, counts,
                tokens * top, E, tile_rows, offsets, tiles, n_tiles, src_of_row, row_of, E - identity);
    VX_LAUNCH_CHECK();
    return VX_OK;
}

// ---- grouped product on the CUDA cores: any sizes, float32 sums over k ascending ----
#define MG_BM 64
#define MG_BN 64
#define MG_BK 16

template <typename TA, typename TC>
__global__ void __launch_bounds__(256)
moe_gemm_simt_kernel(const TA* __restrict__ A, int lda, const int* __restrict__ src_of_row, int src_div,
                     const TA* __restrict__ W, const int* __restrict__ tiles, const int* __restrict__ n_tiles,
                     TC* __restrict__ C, int ldc, int N, int K, int gated, int act) {
    pdl_wait();
    pdl_trigger();
    if ((int)blockIdx.y >= n_tiles[0]) return;
    __shared__ float As[MG_BK][MG_BM + 1];
    __shared__ float Ws[MG_BK][MG_BN + 1];
    __shared__ int src_s[MG_BM];
    const int e = tiles[3 * blockIdx.y], row0 = tiles[3 * blockIdx.y + 1], rows = tiles[3 * blockIdx.y + 2];
    const TA* We = W + (size_t)e * N * K;
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const int n0 = blockIdx.x * MG_BN;
    const int lk = tid & 15, lr = tid >> 4;
    if (tid < MG_BM) {
        const int p = row0 + tid;
        src_s[tid] = tid < rows ? (src_of_row ? src_of_row[p] / src_div : p) : -1;
    }
    __syncthreads();
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    for (int k0 = 0; k0 < K; k0 += MG_BK) {
        const int k = k0 + lk;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int r = lr + 16 * i;
            const int s = src_s[r], n = n0 + r;
            As[lk][r] = (s >= 0 && k < K) ? to_f32(A[(size_t)s * lda + k]) : 0.f;
            Ws[lk][r] = (n < N && k < K) ? to_f32(We[(size_t)n * K + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < MG_BK; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty + 16 * i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = Ws[kk][tx + 16 * j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = ty + 16 * i;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx + 16 * j;
            float v = acc[i][j];
            if (gated) {
                // columns come as 8 gates, then their 8 ups: the up of this thread's gate is 8 lanes on
                const float up = __shfl_xor_sync(0xffffffffu, v, 8);
                if (tx < 8 && r < rows && n < N)
                    C[(size_t)(row0 + r) * ldc + (n >> 4) * 8 + tx] = from_f32<TC>(activation(v, act) * up);
            } else if (r < rows && n < N) {
                C[(size_t)(row0 + r) * ldc + n] = from_f32<TC>(v);
            }
        }
    }
}

// ---- grouped product on the tensor cores (bfloat16 operands, float32 accumulators) ----
// A block of 4 warps owns a tile of 64 rows x 64 columns; warp w takes rows 32 * (w & 1) and
// columns 32 * (w >> 1).  k runs in steps of 64 (128 bytes of every row) through three
// shared-memory stages filled by 16-byte asynchronous copies, two of them in flight while one is
// multiplied (rows that do not exist are zero).  K a multiple of 8.
#define MT_BM 64
#define MT_BN 64
#define MT_BK 64
#define MT_STAGES 3
#define MT_LD (MT_BK + 8)   // (a row of 144 bytes: the 8 rows of a matrix load miss each other's banks)
#define MT_SMEM (MT_STAGES * (MT_BM + MT_BN) * MT_LD * 2)

template <typename TC>
__global__ void __launch_bounds__(128)
moe_gemm_mma_kernel(const bf16* __restrict__ A, int lda, const int* __restrict__ src_of_row, int src_div,
                    const bf16* __restrict__ W, const int* __restrict__ tiles, const int* __restrict__ n_tiles,
                    TC* __restrict__ C, int ldc, int N, int K, int gated, int act) {
    extern __shared__ __align__(16) unsigned char mt_smem[];
    typedef bf16 (*Tile)[MT_BM][MT_LD];
    Tile As = reinterpret_cast<Tile>(mt_smem);
    Tile Ws = reinterpret_cast<Tile>(mt_smem + MT_STAGES * MT_BM * MT_LD * 2);
    __shared__ int src_s[MT_BM];
    pdl_wait();
    pdl_trigger();
    if ((int)blockIdx.y >= n_tiles[0]) return;
    const int e = tiles[3 * blockIdx.y], row0 = tiles[3 * blockIdx.y + 1], rows = tiles[3 * blockIdx.y + 2];
    const bf16* We = W + (size_t)e * N * K;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n0 = blockIdx.x * MT_BN;
    if (tid < MT_BM) {
        const int p = row0 + tid;
        src_s[tid] = tid < rows ? (src_of_row ? src_of_row[p] / src_div : p) : -1;
    }
    __syncthreads();
    const int wm = (warp & 1) * 32, wn = (warp >> 1) * 32;
    float acc[2][4][4];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[i][j][c] = 0.f;

    auto load_stage = [&](int stage, int k0) {
        // 64 rows x 8 chunks of 8 elements per operand; 128 threads take 4 chunks of each
#pragma unroll
        for (int it = 0; it < 4; ++it) {
            const int idx = tid + it * 128;
            const int r = idx >> 3, ck = (idx & 7) * 8;
            const int k = k0 + ck;
            bf16* da = &As[stage][r][ck];
            const int s = src_s[r];
            if (s >= 0 && k < K) cp_async16(da, A + (size_t)s * lda + k);
            else *reinterpret_cast<uint4*>(da) = make_uint4(0, 0, 0, 0);
            bf16* dw = &Ws[stage][r][ck];
            const int n = n0 + r;
            if (n < N && k < K) cp_async16(dw, We + (size_t)n * K + k);
            else *reinterpret_cast<uint4*>(dw) = make_uint4(0, 0, 0, 0);
        }
        cp_async_commit();
    };

    const int nk = (K + MT_BK - 1) / MT_BK;
#pragma unroll
    for (int st = 0; st < MT_STAGES - 1; ++st) {
        if (st < nk) load_stage(st, st * MT_BK); else cp_async_commit();
    }
    for (int kb = 0; kb < nk; ++kb) {
        const int cur = kb % MT_STAGES;
        cp_async_wait<MT_STAGES - 2>();   // all but the newest groups have landed: stage `cur` is there
        __syncthreads();      // ... for every thread's copies, and everybody is done with the stage filled next
        if (kb + MT_STAGES - 1 < nk) load_stage((kb + MT_STAGES - 1) % MT_STAGES, (kb + MT_STAGES - 1) * MT_BK);
        else cp_async_commit();
#pragma unroll
        for (int ks = 0; ks < MT_BK; ks += 16) {
            unsigned a[2][4], b[4][2];
#pragma unroll
            for (int i = 0; i < 2; ++i)
                ldmatrix_x4(a[i][0], a[i][1], a[i][2], a[i][3], &As[cur][wm + 16 * i + (lane & 15)][ks + (lane >> 4) * 8]);
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                // two n-tiles of 8 columns at once: matrices (n 0-7, k 0-7), (n 0-7, k 8-15), (n 8-15, k 0-7), (n 8-15, k 8-15)
                unsigned r0, r1, r2, r3;
                ldmatrix_x4(r0, r1, r2, r3, &Ws[cur][wn + 16 * j + (lane & 7) + ((lane >> 4) << 3)][ks + ((lane >> 3) & 1) * 8]);
                b[2 * j][0] = r0; b[2 * j][1] = r1; b[2 * j + 1][0] = r2; b[2 * j + 1][1] = r3;
            }
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) mma_bf16(acc[i][j], a[i], b[j][0], b[j][1]);
        }
    }
    // accumulator layout of m16n8: c0,c1 at (row lane/4, cols 2*(lane%4), +1); c2,c3 eight rows further down
#pragma unroll
    for (int i = 0; i < 2; ++i) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int r = wm + 16 * i + (lane >> 2) + 8 * half;
            if (r >= rows) continue;
            TC* crow = C + (size_t)(row0 + r) * ldc;
            if (gated) {
#pragma unroll
                for (int j = 0; j < 4; j += 2) {   // n-tile j: 8 gates, n-tile j + 1: their ups
                    const int n = n0 + wn + 8 * j + 2 * (lane & 3);
#pragma unroll
                    for (int c = 0; c < 2; ++c)
                        if (n + c < N)
                            crow[((n + c) >> 4) * 8 + ((n + c) & 7)] =
                                from_f32<TC>(activation(acc[i][j][2 * half + c], act) * acc[i][j + 1][2 * half + c]);
                }
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int n = n0 + wn + 8 * j + 2 * (lane & 3);
#pragma unroll
                    for (int c = 0; c < 2; ++c)
                        if (n + c < N) crow[n + c] = from_f32<TC>(acc[i][j][2 * half + c]);
                }
            }
        }
    }
}

// The same for steps of few tokens (decode): row tiles of 16, so that a step's handful of rows per expert costs
// one m16 tile of products, not four; a block of 4 warps owns 16 rows x 64 columns (16 columns a warp) and
// streams its 64 rows of W through four stages.
#define MS_BM 16
#define MS_STAGES 4
#define MS_SMEM (MS_STAGES * (MS_BM + MT_BN) * MT_LD * 2)

template <typename TC>
__global__ void __launch_bounds__(128)
moe_gemm_mma16_kernel(const bf16* __restrict__ A, int lda, const int* __restrict__ src_of_row, int src_div,
                      const bf16* __restrict__ W, const int* __restrict__ tiles, const int* __restrict__ n_tiles,
                      TC* __restrict__ C, int ldc, int N, int K, int gated, int act) {
    extern __shared__ __align__(16) unsigned char ms_smem[];
    typedef bf16 (*TileA)[MS_BM][MT_LD];
    typedef bf16 (*TileW)[MT_BN][MT_LD];
    TileA As = reinterpret_cast<TileA>(ms_smem);
    TileW Ws = reinterpret_cast<TileW>(ms_smem + MS_STAGES * MS_BM * MT_LD * 2);
    __shared__ int src_s[MS_BM];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n0 = blockIdx.x * MT_BN;
    pdl_wait();
    pdl_trigger();
    if ((int)blockIdx.y >= n_tiles[0]) return;
    const int e = tiles[3 * blockIdx.y], row0 = tiles[3 * blockIdx.y + 1], rows = tiles[3 * blockIdx.y + 2];
    const bf16* We = W + (size_t)e * N * K;
    if (tid < MS_BM) {
        const int p = row0 + tid;
        src_s[tid] = tid < rows ? (src_of_row ? src_of_row[p] / src_div : p) : -1;
    }
    __syncthreads();
    const int wn = warp * 16;
    float acc[2][4];
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[j][c] = 0.f;
    auto load_stage = [&](int stage, int k0) {
        {   // 16 rows x 8 chunks of A: one a thread
            const int r = tid >> 3, ck = (tid & 7) * 8;
            bf16* da = &As[stage][r][ck];
            const int s = src_s[r];
            if (s >= 0 && k0 + ck < K) cp_async16(da, A + (size_t)s * lda + k0 + ck);
            else *reinterpret_cast<uint4*>(da) = make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int it = 0; it < 4; ++it) {   // 64 rows x 8 chunks of W: four a thread
            const int idx = tid + it * 128;
            const int r = idx >> 3, ck = (idx & 7) * 8;
            bf16* dw = &Ws[stage][r][ck];
            if (n0 + r < N && k0 + ck < K) cp_async16(dw, We + (size_t)(n0 + r) * K + k0 + ck);
            else *reinterpret_cast<uint4*>(dw) = make_uint4(0, 0, 0, 0);
        }
        cp_async_commit();
    };
    const int nk = (K + MT_BK - 1) / MT_BK;
#pragma unroll
    for (int st = 0; st < MS_STAGES - 1; ++st) {
        if (st < nk) load_stage(st, st * MT_BK); else cp_async_commit();
    }
    for (int kb = 0; kb < nk; ++kb) {
        const int cur = kb % MS_STAGES;
        cp_async_wait<MS_STAGES - 2>();
        __syncthreads();
        if (kb + MS_STAGES - 1 < nk) load_stage((kb + MS_STAGES - 1) % MS_STAGES, (kb + MS_STAGES - 1) * MT_BK);
        else cp_async_commit();
#pragma unroll
        for (int ks = 0; ks < MT_BK; ks += 16) {
            unsigned a[4], r0, r1, r2, r3;
            ldmatrix_x4(a[0], a[1], a[2], a[3], &As[cur][lane & 15][ks + (lane >> 4) * 8]);
            ldmatrix_x4(r0, r1, r2, r3, &Ws[cur][wn + (lane & 7) + ((lane >> 4) << 3)][ks + ((lane >> 3) & 1) * 8]);
            mma_bf16(acc[0], a, r0, r1);
            mma_bf16(acc[1], a, r2, r3);
        }
    }
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int r = (lane >> 2) + 8 * half;
        if (r >= rows) continue;
        TC* crow = C + (size_t)(row0 + r) * ldc;
        const int n = n0 + wn + 2 * (lane & 3);
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            if (gated) {   // the warp's 16 columns: 8 gates, then their 8 ups
                if (n + c < N)
                    crow[((n + c) >> 4) * 8 + ((n + c) & 7)] =
                        from_f32<TC>(activation(acc[0][2 * half + c], act) * acc[1][2 * half + c]);
            } else {
                if (n + c < N) crow[n + c] = from_f32<TC>(acc[0][2 * half + c]);
                if (n + 8 + c < N) crow[n + 8 + c] = from_f32<TC>(acc[1][2 * half + c]);
            }
        }
    }
}

// in_dtype: A and W; out_dtype: C.  `tensor_cores`: the bfloat16 kernel (K a multiple of 8,
// 16-byte aligned rows); else the multiply-add kernel.  max_tiles bounds the tiles of any step.
// tile_rows: 64, or 16 (tensor cores only) for steps of few tokens.
extern "C" int vx_moe_gemm(const void* A, int lda, const int* src_of_row, int src_div, const void* W, const int* tiles,
                           const int* n_tiles, int max_tiles, void* C, int ldc, int N, int K, int gated, int act,
                           int in_dtype, int out_dtype, int tensor_cores, int tile_rows, cudaStream_t stream) {
    if (max_tiles <= 0 || N <= 0) return VX_OK;
    if (K <= 0 || lda < K || src_div <= 0 || (gated && N % 16)) return VX_ERR_SHAPE;
    if (max_tiles > 65535) return VX_ERR_LIMIT;
    if (tile_rows != MT_BM && !(tile_rows == MS_BM && tensor_cores)) return VX_ERR_SHAPE;
    dim3 grid((N + MG_BN - 1) / MG_BN, max_tiles);
    if (tensor_cores && tile_rows == MS_BM) {
        if (in_dtype != VX_BF16) return VX_ERR_DTYPE;
        if (K % 8 || lda % 8 || (((uintptr_t)A) | ((uintptr_t)W)) & 15) return VX_ERR_ALIGN;
        static bool conf_b[VX_MAX_DEVICES], conf_f[VX_MAX_DEVICES];
        if (int rc = out_dtype == VX_BF16 ? vx_configure_smem(moe_gemm_mma16_kernel<bf16>, MS_SMEM, conf_b)
                                          : vx_configure_smem(moe_gemm_mma16_kernel<float>, MS_SMEM, conf_f)) return rc;
        if (out_dtype == VX_BF16)
            VX_LAUNCH_K(VX_K_GEMM, (moe_gemm_mma16_kernel<bf16>), grid, 128, MS_SMEM, stream, (const bf16*)A, lda, src_of_row,
                        src_div, (const bf16*)W, tiles, n_tiles, (bf16*)C, ldc, N, K, gated, act);
        else if (out_dtype == VX_F32)
            VX_LAUNCH_K(VX_K_GEMM, (moe_gemm_mma16_kernel<float>), grid, 128, MS_SMEM, stream, (const bf16*)A, lda, src_of_row,
                        src_div, (const bf16*)W, tiles, n_tiles, (float*)C, ldc, N, K, gated, act);
        else
            return VX_ERR_DTYPE;
    } else if (tensor_cores) {
        if (in_dtype != VX_BF16) return VX_ERR_DTYPE;
        if (K % 8 || lda % 8 || (((uintptr_t)A) | ((uintptr_t)W)) & 15) return VX_ERR_ALIGN;
        static bool configured_b[VX_MAX_DEVICES], configured_f[VX_MAX_DEVICES];
        if (int rc = out_dtype == VX_BF16 ? vx_configure_smem(moe_gemm_mma_kernel<bf16>, MT_SMEM, configured_b)
                                          : vx_configure_smem(moe_gemm_mma_kernel<float>, MT_SMEM, configured_f)) return rc;
        if (out_dtype == VX_BF16)
            VX_LAUNCH_K(VX_K_GEMM, (moe_gemm_mma_kernel<bf16>), grid, 128, MT_SMEM, stream, (const bf16*)A, lda, src_of_row, src_div,
                        (const bf16*)W, tiles, n_tiles, (bf16*)C, ldc, N, K, gated, act);
        else if (out_dtype == VX_F32)
            VX_LAUNCH_K(VX_K_GEMM, (moe_gemm_mma_kernel<float>), grid, 128, MT_SMEM, stream, (const bf16*)A, lda, src_of_row, src_div,
                        (const bf16*)W, tiles, n_tiles, (float*)C, ldc, N, K, gated, act);
        else
            return VX_ERR_DTYPE;
    } else if (in_dtype == VX_F32 && out_dtype == VX_F32)
        VX_LAUNCH_K(VX_K_GEMM, (moe_gemm_simt_kernel<float, float>), grid, 256, 0, stream, (const float*)A, lda, src_of_row,
                    src_div, (const float*)W, tiles, n_tiles, (float*)C, ldc, N, K, gated, act);
    else if (in_dtype == VX_BF16 && out_dtype == VX_BF16)
        VX_LAUNCH_K(VX_K_GEMM, (moe_gemm_simt_kernel<bf16, bf16>), grid, 256, 0, stream, (const bf16*)A, lda, src_of_row,
                    src_div, (const bf16*)W, tiles, n_tiles, (bf16*)C, ldc, N, K, gated, act);
    else if (in_dtype == VX_BF16 && out_dtype == VX_F32)
        VX_LAUNCH_K(VX_K_GEMM, (moe_gemm_simt_kernel<bf16, float>), grid, 256, 0, stream, (const bf16*)A, lda, src_of_row,
                    src_div, (const bf16*)W, tiles, n_tiles, (float*)C, ldc, N, K, gated, act);
    else
        return VX_ERR_DTYPE;
    VX_LAUNCH_CHECK();
    return VX_OK;
}

// out[p, :] = x[src_of_row[p] / div, :] for the rows p of expert order (16 bytes a thread and step): the
// activations in the order the tcgen05 grouped product reads them by TMA.
__global__ void moe_gather_rows_kernel(const uint4* __restrict__ x, int ldx16, const int* __restrict__ src_of_row, int div,
                                       uint4* __restrict__ out, int chunks) {
    pdl_wait();
    pdl_trigger();
    const int p = blockIdx.x;
    const uint4* src = x + (size_t)(src_of_row[p] / div) * ldx16;
    for (int c = threadIdx.x; c < chunks; c += blockDim.x) out[(size_t)p * chunks + c] = src[c];
}

extern "C" int vx_moe_gather_rows(const void* x, int ldx, const int* src_of_row, int div, void* out, int rows, int width,
                                  cudaStream_t stream) {
    if (rows <= 0) return VX_OK;
    if (width <= 0 || width % 8 || ldx % 8 || div <= 0) return VX_ERR_SHAPE;
    if ((((uintptr_t)x) | ((uintptr_t)out)) & 15) return VX_ERR_ALIGN;
    VX_LAUNCH_K(VX_K_ELEMENTWISE, moe_gather_rows_kernel, rows, 128, 0, stream, (const uint4*)x, ldx / 8, src_of_row, div,
                (uint4*)out, width / 8);
    VX_LAUNCH_CHECK();
    return VX_OK;
}

// out[t, :] = sum over k (ascending) of weight[t, k] * y[row_of[t * top + k], :] (+ shared[t, :]).
template <typename T, typename TY>
__global__ void moe_combine_kernel(const TY* __restrict__ y, const int* __restrict__ row_of,
                                   const float* __restrict__ weight, const T* __restrict__ shared_out,
                                   T* __restrict__ out, int width, int top, const int* __restrict__ chosen, int n_real,
                                   const T* __restrict__ h, int ldh, const float* __restrict__ shared_gate) {
    __shared__ int row_s[MOE_MAX_TOP];
    __shared__ float w_s[MOE_MAX_TOP];
    pdl_wait();
    pdl_trigger();
    const int t = blockIdx.x;
    if (threadIdx.x < top) {
        // (a negative row: the assignment went to an identity expert, whose output is the token's own row)
        const bool same = chosen && chosen[(size_t)t * top + threadIdx.x] >= n_real;
        row_s[threadIdx.x] = same ? -1 : row_of[(size_t)t * top + threadIdx.x];
        w_s[threadIdx.x] = weight[(size_t)t * top + threadIdx.x];
    }
    __syncthreads();
    const float g = shared_gate ? shared_gate[t] : 1.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float s = 0.f;
        for (int k = 0; k < top; ++k)
            s = fmaf(w_s[k], row_s[k] < 0 ? to_f32(h[(size_t)t * ldh + i]) : to_f32(y[(size_t)row_s[k] * width + i]), s);
        if (shared_out) s = fmaf(g, to_f32(shared_out[(size_t)t * width + i]), s);
        out[(size_t)t * width + i] = from_f32<T>(s);
    }
}

// y_dtype: the element type of the experts' rows (float32, or bfloat16 from the tcgen05 product).
// With `chosen` and `n_real`, assignments to outputs >= n_real take the token's own row of `h` [tokens, ldh] instead of
// a row of `y`; with `shared_gate` the shared expert's row is multiplied by shared_gate[t].
extern "C" int vx_moe_combine(const void* y, const int* row_of, const float* weight, const void* shared_out, void* out,
                              int tokens, int width, int top, int dtype, int y_dtype, const int* chosen, int n_real,
                              const void* h, int ldh, const float* shared_gate, cudaStream_t stream) {
    if (tokens <= 0) return VX_OK;
    if (width <= 0 || top <= 0 || (chosen && !h)) return VX_ERR_SHAPE;
    if (top > MOE_MAX_TOP) return VX_ERR_LIMIT;
    const int threads = width >= 1024 ? 256 : 128;
    if (dtype == VX_F32 && y_dtype == VX_F32)
        VX_LAUNCH_K(VX_K_ELEMENTWISE, (moe_combine_kernel<float, float>), tokens, threads, 0, stream, (const float*)y, row_of,
                    weight, (const float*)shared_out, (float*)out, width, top, chosen, n_real, (const float*)h, ldh, shared_gate);
    else if (dtype == VX_BF16 && y_dtype == VX_F32)
        VX_LAUNCH_K(VX_K_ELEMENTWISE, (moe_combine_kernel<bf16, float>), tokens, threads, 0, stream, (const float*)y, row_of,
                    weight, (const bf16*)shared_out, (bf16*)out, width, top, chosen, n_real, (const bf16*)h, ldh, shared_gate);
    else if (dtype == VX_BF16 && y_dtype == VX_BF16)
        VX_LAUNCH_K(VX_K_ELEMENTWISE, (moe_combine_kernel<bf16, bf16>), tokens, threads, 0, stream, (const bf16*)y, row_of,
                    weight, (const bf16*)shared_out, (bf16*)out, width, top, chosen, n_real, (const bf16*)h, ldh, shared_gate);
    else
        return VX_ERR_DTYPE;
    VX_LAUNCH_CHECK();
    return VX_OK;
}
