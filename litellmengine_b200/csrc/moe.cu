// Routed experts (mixture of experts): the router, and the experts' activation with the routing weights.
//
// moe_route_kernel   per token: logits z = W_r x in 32-bit (x may be the compute dtype's rounding of the
//                    normed stream; W_r is held in float32), scores s = sigmoid(z).  Experts form `groups`
//                    equal groups of neighbours; a group's score is the sum of its two largest scores (of
//                    its one score when a group is one expert) and only experts of the `keep` best groups
//                    may be chosen (groups = 0: no such limit).  The `top` largest allowed scores are
//                    chosen (ties go to the lower index); their weights are s / (sum of the chosen s +
//                    1e-20) * route_scale.  Written as a dense row of float32 weights [experts] (zero for
//                    experts that were not chosen) and, optionally, as the lists ids [top], weights [top].
//                    `softmax` 1: the scores are softmax(z) over all router outputs instead.  `correction`
//                    (float32 [router outputs], optional) is added to a score for the CHOICE only; the weights
//                    are made of the scores themselves.  The last `identity` router outputs stand for no
//                    expert at all: a token that picks one gets its own input back times the weight.  Those
//                    have no column in the dense row (it has E - identity columns), their place in the lists
//                    holds id -1 and weight 0, and the sum of their weights goes to `idw` [tokens].
//                    The experts' activation: g = min(gate, limit), u = clamp(up, -limit, limit),
//                    w * g * sigmoid(alpha g) * (u + up_shift); limit = infinity, alpha = 1, up_shift = 0 is
//                    the plain silu(gate) * up.
// moe_act_kernel     from the float32 product [T, experts * 2 * ff] of the token rows with every expert's
//                    [gate; up] matrix: act[t, e*ff + f] = w[t, e] * g * sigmoid(alpha g) * (u + 1) with
//                    g = min(gate, limit), u = clamp(up, -limit, limit), in the compute dtype, zero where
//                    w[t, e] is zero.  The experts' down matrices stand side by side along the input axis,
//                    so ONE product of `act` with them is the weighted sum of the chosen experts' outputs.
#include "common.cuh"
#include <math_constants.h>

#define MOE_ROUTE_THREADS 256
#define MOE_ROUTE_TOKENS 4        // tokens a block takes: the router's matrix is read once for all of them

template <typename TX>
__global__ void moe_route_kernel(const TX* __restrict__ x, const float* __restrict__ wr, float* __restrict__ dense,
                                 int32_t* __restrict__ ids, float* __restrict__ weights, int num_tokens, int W, int E,
                                 int top, int groups, int keep, float route_scale, int vec, int softmax,
                                 const float* __restrict__ correction, int identity, float* __restrict__ idw) {
    pdl_begin();
    extern __shared__ float smem[];
    const int G = groups > 0 ? groups : 1;
    float* xs = smem;                                   // [TOKENS][W]
    float* score = xs + MOE_ROUTE_TOKENS * W;           // [TOKENS][E]
    float* gscore = score + MOE_ROUTE_TOKENS * E;       // [TOKENS][G]
    int* allowed = reinterpret_cast<int*>(gscore + MOE_ROUTE_TOKENS * G);      // [TOKENS][E]
    const long long t0 = static_cast<long long>(blockIdx.x) * MOE_ROUTE_TOKENS;
    const int nt = static_cast<int>(min(static_cast<long long>(MOE_ROUTE_TOKENS), num_tokens - t0));
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (vec) {                                          // sixteen-byte loads of the tokens' rows
        for (int i = tid * 8; i < nt * W; i += blockDim.x * 8) {
            float v[8];
            load8(x + t0 * W + i, v);
#pragma unroll
            for (int u = 0; u < 8; ++u) xs[i + u] = v[u];
        }
    } else {
        for (int i = tid; i < nt * W; i += blockDim.x) xs[i] = to_f32(x[t0 * W + i]);
    }
    __syncthreads();
    for (int e = warp; e < E; e += MOE_ROUTE_THREADS / 32) {       // a warp an expert: its row against the block's tokens
        const float* w = wr + static_cast<size_t>(e) * W;
        float dot[MOE_ROUTE_TOKENS];
#pragma unroll
        for (int k = 0; k < MOE_ROUTE_TOKENS; ++k) dot[k] = 0.0f;
        if (vec) {                                      // sixteen bytes of the row a lane and trip, four trips in flight
#pragma unroll 4
            for (int i = lane * 4; i < W; i += 128) {
                const float4 wv = *reinterpret_cast<const float4*>(w + i);
#pragma unroll
                for (int k = 0; k < MOE_ROUTE_TOKENS; ++k) {      // rows past nt hold stale data: never used
                    const float4 xv = *reinterpret_cast<const float4*>(xs + k * W + i);
                    dot[k] += wv.x * xv.x + wv.y * xv.y + wv.z * xv.z + wv.w * xv.w;
                }
            }
        } else {
            for (int i = lane; i < W; i += 32) {
                const float wv = w[i];
#pragma unroll
                for (int k = 0; k < MOE_ROUTE_TOKENS; ++k) dot[k] += wv * xs[k * W + i];
            }
        }
#pragma unroll
        for (int k = 0; k < MOE_ROUTE_TOKENS; ++k) {
            const float d = warp_sum(dot[k]);
            if (lane == 0 && k < nt) score[k * E + e] = softmax ? d : 1.0f / (1.0f + expf(-d));
        }
    }
    __syncthreads();
    if (softmax) {                                   // a warp a token: maximum, exponentials, their sum
        if (warp < nt) {
            float* sc = score + warp * E;
            float top_z = -CUDART_INF_F;
            for (int e = lane; e < E; e += 32) top_z = fmaxf(top_z, sc[e]);
            top_z = warp_max(top_z);
            float sum = 0.0f;
            for (int e = lane; e < E; e += 32) {
                const float p = expf(sc[e] - top_z);
                sc[e] = p;
                sum += p;
            }
            sum = warp_sum(sum);
            for (int e = lane; e < E; e += 32) sc[e] = sc[e] / sum;
        }
        __syncthreads();
    }
    const int per = groups > 0 ? E / groups : E;
    for (int idx = tid; idx < nt * G && groups > 0; idx += blockDim.x) {
        const int k = idx / G, g = idx - k * G;
        float a = -CUDART_INF_F, b = -CUDART_INF_F;  // the two largest
        for (int j = 0; j < per; ++j) {
            const float sc = score[k * E + g * per + j] + (correction ? correction[g * per + j] : 0.0f);
            if (sc > a) { b = a; a = sc; }
            else if (sc > b) b = sc;
        }
        gscore[idx] = per > 1 ? a + b : a;
    }
    const int real = E - identity;                   // the experts that are feed-forwards: the dense row's columns
    for (int idx = tid; idx < nt * E; idx += blockDim.x) allowed[idx] = groups > 0 ? 0 : 1;
    for (int idx = tid; idx < nt * real; idx += blockDim.x) dense[t0 * real + idx] = 0.0f;
    __syncthreads();
    if (tid < nt) {                                  // one thread a token walks the choices (a few dozen steps)
        const int k = tid;
        const long long t = t0 + k;
        float* sc = score + k * E;
        int* ok = allowed + k * E;
        for (int n = 0; n < keep && groups > 0; ++n) {      // the best groups, ties to the lower index
            int best = -1;
            float bs = -CUDART_INF_F;
            for (int g = 0; g < groups; ++g)
                if (gscore[k * G + g] > bs) { bs = gscore[k * G + g]; best = g; }
            if (best < 0) break;
            gscore[k * G + best] = -CUDART_INF_F;
            for (int j = 0; j < per; ++j) ok[best * per + j] = 1;
        }
        float total = 0.0f;
        int chosen[64];
        for (int n = 0; n < top; ++n) {
            int best = -1;
            float bs = -CUDART_INF_F;
            for (int e = 0; e < E; ++e) {
                const float cv = sc[e] + (correction ? correction[e] : 0.0f);       // the choice's score; the weight's is sc
                if (ok[e] && cv > bs) { bs = cv; best = e; }
            }
            chosen[n] = best;
            if (best >= 0) {
                ok[best] = 0;
                total += sc[best];
            }
        }
        const float inv = route_scale / (total + 1e-20f);
        float own = 0.0f;                            // what the token gets of its own input
        for (int n = 0; n < top; ++n) {
            const int e = chosen[n];
            const float w = e >= 0 ? sc[e] * inv : 0.0f;
            const bool expert = e >= 0 && e < real;
            if (expert) dense[t * real + e] = w;
            else if (e >= 0) own += w;
            if (ids) {
                ids[t * top + n] = expert ? e : -1;
                weights[t * top + n] = expert ? w : 0.0f;
            }
        }
        if (idw) idw[t] = own;
    }
}

extern "C" int llm_moe_route(const void* x, int x_dtype, const float* wr, float* dense, int32_t* ids, float* weights,
                             int num_tokens, int W, int E, int top, int groups, int keep, float route_scale,
                             int softmax, const float* correction, int identity, float* idw, uintptr_t stream) {
    if (num_tokens <= 0) return LLM_OK;
    if (identity < 0 || identity >= E || (identity > 0 && !idw)) return LLM_REFUSED_SIZE;
    if (W <= 0 || E <= 0 || top <= 0 || top > E || top > 64 || groups < 0) return LLM_REFUSED_SIZE;
    if (groups > 0 && (E % groups || keep <= 0 || keep > groups || keep * (E / groups) < top)) return LLM_REFUSED_SIZE;
    const size_t smem = MOE_ROUTE_TOKENS * (static_cast<size_t>(W) + 2 * E + (groups > 0 ? groups : 1)) * sizeof(float);
    if (smem > 200 * 1024) return LLM_REFUSED_SIZE;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    const dim3 grid((num_tokens + MOE_ROUTE_TOKENS - 1) / MOE_ROUTE_TOKENS);
    const int vec = W % 8 == 0 && aligned16(x) && aligned16(wr);
#define LAUNCH(TX)                                                                                                  \
    do {                                                                                                            \
        auto kern = moe_route_kernel<TX>;                                                                           \
        if (smem > 48 * 1024) {                                                                                     \
            const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,           \
                                                       static_cast<int>(smem));                                     \
            if (e != cudaSuccess) return static_cast<int>(e);                                                       \
        }                                                                                                           \
        launch_pdl(kern, grid, dim3(MOE_ROUTE_THREADS), smem, s, static_cast<const TX*>(x), wr, dense, ids, weights,  \
                   num_tokens, W, E, top, groups, keep, route_scale, vec, softmax, correction, identity, idw);      \
    } while (0)
    if (x_dtype == LLM_DT_F32) LAUNCH(float);
    else if (x_dtype == LLM_DT_BF16) LAUNCH(bf16);
    else return LLM_REFUSED_DTYPE;
#undef LAUNCH
    return launch_status();
}

// An expert's activation: the clamped gate through g * sigmoid(alpha g), times the clamped up value plus `shift`.
__device__ __forceinline__ float moe_activate(float g, float u, float limit, float alpha, float shift) {
    const float gc = fminf(g, limit), uc = fminf(fmaxf(u, -limit), limit);
    return (gc / (1.0f + expf(-alpha * gc))) * (uc + shift);
}
__device__ __forceinline__ void moe_store4(float* p, const float (&v)[4]) { *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]); }
__device__ __forceinline__ void moe_store4(bf16* p, const float (&v)[4]) {
    uint2 raw;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
    h[0] = __floats2bfloat162_rn(v[0], v[1]);
    h[1] = __floats2bfloat162_rn(v[2], v[3]);
    *reinterpret_cast<uint2*>(p) = raw;
}

// One block row per (token, expert): the token's weight for the expert is read once; a thread makes VEC
// neighbouring features (VEC = 4: sixteen-byte loads of the gate and up values, which are only touched
// for experts that were chosen; the others' columns are zeroed).
template <typename TO, int VEC>
__global__ void moe_act_kernel(const float* __restrict__ gu, int parts, long long part_stride,
                               const float* __restrict__ dense, TO* __restrict__ act, int E, int ff, float limit,
                               float alpha, float shift) {
    pdl_begin();
    const long long pair = blockIdx.x;                  // token * E + expert
    const int f = (blockIdx.y * blockDim.x + threadIdx.x) * VEC;
    if (f >= ff) return;
    const float w = dense[pair];
    float out[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    if (w != 0.0f) {
        const float* p = gu + pair * 2 * ff;
        float g[4] = {0.0f, 0.0f, 0.0f, 0.0f}, u[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        for (int k = 0; k < parts; ++k) {                   // the product may come as its k-splits
            if (VEC == 4) {
                const float4 a = *reinterpret_cast<const float4*>(p + k * part_stride + f);
                const float4 b = *reinterpret_cast<const float4*>(p + k * part_stride + ff + f);
                g[0] += a.x; g[1] += a.y; g[2] += a.z; g[3] += a.w;
                u[0] += b.x; u[1] += b.y; u[2] += b.z; u[3] += b.w;
            } else {
                g[0] += p[k * part_stride + f];
                u[0] += p[k * part_stride + ff + f];
            }
        }
#pragma unroll
        for (int c = 0; c < VEC; ++c) out[c] = w * moe_activate(g[c], u[c], limit, alpha, shift);
    }
    TO* o = act + pair * ff + f;
    if (VEC == 4) moe_store4(o, out);
    else o[0] = from_f32<TO>(out[0]);
}

extern "C" int llm_moe_act(const float* gu, int parts, long long part_stride, const float* dense, void* act,
                           int act_dtype, int num_tokens, int E, int ff, float limit, float alpha, float shift,
                           uintptr_t stream) {
    if (num_tokens <= 0) return LLM_OK;
    if (E <= 0 || ff <= 0 || !(limit > 0.0f)) return LLM_REFUSED_SIZE;
    const long long pairs = static_cast<long long>(num_tokens) * E;
    if (pairs > 0x7fffffffLL) return LLM_REFUSED_SIZE;
    if (parts < 1) parts = 1;
    const bool vec = ff % 4 == 0 && aligned16(gu) && aligned16(act) && part_stride % 4 == 0;
    const int per_block = 128 * (vec ? 4 : 1);
    const dim3 grid(static_cast<unsigned>(pairs), (ff + per_block - 1) / per_block);
    if (grid.y > 65535) return LLM_REFUSED_SIZE;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
#define LAUNCH(TO, V)                                                                                          \
    launch_pdl((moe_act_kernel<TO, V>), grid, dim3(128), 0, s, gu, parts, part_stride, dense, static_cast<TO*>(act), E, ff, \
               limit, alpha, shift)
    if (act_dtype == LLM_DT_F32) { if (vec) LAUNCH(float, 4); else LAUNCH(float, 1); }
    else if (act_dtype == LLM_DT_BF16) { if (vec) LAUNCH(bf16, 4); else LAUNCH(bf16, 1); }
    else return LLM_REFUSED_DTYPE;
#undef LAUNCH
    return launch_status();
}

// ---- steps of few tokens: only the chosen experts' weights are read --------------------------------------
// For a decode step the dense form above would stream every expert's matrices for a handful of tokens.
// These two kernels walk the (token, chosen expert) pairs instead; a warp makes one output feature at a
// time as a dot product over 16-byte loads of the weight row against the token's row held in shared
// memory (32-bit accumulation), so the chosen experts' bytes bound them.
//   moe_gate_up_sparse_kernel   act[pair, f] = w * g * sigmoid(alpha g) * (u + 1) for pair = (token, k-th choice)
//   moe_down_sparse_kernel      out[token, n] = sum over the token's choices of W_down[e][n, :] . act[pair, :]
// Weights: `w_gate_up` [E * 2 * ff, W] (per expert ff gate rows, then ff up rows) and `w_down` [W, E * ff].
#define MOE_SPARSE_WARPS 8
#define MOE_SPARSE_FEATURES 8

// Two rows against one vector, their loads in flight together.
template <typename TW>
__device__ __forceinline__ void moe_dot2(const TW* __restrict__ w0, const TW* __restrict__ w1, const float* __restrict__ xs,
                                         int n, int lane, bool vec, float& r0, float& r1) {
    float a0 = 0.0f, a1 = 0.0f;
    if (vec) {
        for (int i = lane * 8; i < n; i += 512) {
            float p[8], q[8], p2[8], q2[8];
            const bool more = i + 256 < n;
            load8(w0 + i, p);
            load8(w1 + i, q);
            if (more) {
                load8(w0 + i + 256, p2);
                load8(w1 + i + 256, q2);
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                a0 += p[u] * xs[i + u];
                a1 += q[u] * xs[i + u];
            }
            if (more) {
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    a0 += p2[u] * xs[i + 256 + u];
                    a1 += q2[u] * xs[i + 256 + u];
                }
            }
        }
    } else {
        for (int i = lane; i < n; i += 32) {
            a0 += to_f32(w0[i]) * xs[i];
            a1 += to_f32(w1[i]) * xs[i];
        }
    }
    r0 = warp_sum(a0);
    r1 = warp_sum(a1);
}

template <typename TW>
__device__ __forceinline__ float moe_dot(const TW* __restrict__ w, const float* __restrict__ xs, int n, int lane, bool vec) {
    float acc = 0.0f, acc2 = 0.0f;
    if (vec) {
        for (int i = lane * 8; i < n; i += 1024) {           // up to four sixteen-byte loads in flight a lane
            float p[4][8];
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (i + 256 * j < n) load8(w + i + 256 * j, p[j]);
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (i + 256 * j < n) {
#pragma unroll
                    for (int u = 0; u < 8; u += 2) {
                        acc += p[j][u] * xs[i + 256 * j + u];
                        acc2 += p[j][u + 1] * xs[i + 256 * j + u + 1];
                    }
                }
        }
    } else {
        for (int i = lane; i < n; i += 32) acc += to_f32(w[i]) * xs[i];
    }
    return warp_sum(acc + acc2);
}

template <typename TX, typename TW, typename TO>
__global__ void moe_gate_up_sparse_kernel(const TX* __restrict__ x, const TW* __restrict__ wgu,
                                          const int32_t* __restrict__ ids, const float* __restrict__ weights,
                                          TO* __restrict__ act, int W, int ff, int top, float limit, float alpha, int vec,
                                          float shift) {
    pdl_begin();
    extern __shared__ __align__(16) float xs[];        // [W]
    const int pair = blockIdx.x, t = pair / top;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int e = ids[pair];
    const float wt = weights[pair];
    for (int i = threadIdx.x; i < W; i += blockDim.x) xs[i] = to_f32(x[static_cast<size_t>(t) * W + i]);
    __syncthreads();
    const int f0 = blockIdx.y * MOE_SPARSE_FEATURES;
    for (int f = f0 + warp; f < min(ff, f0 + MOE_SPARSE_FEATURES); f += MOE_SPARSE_WARPS) {
        float out = 0.0f;
        if (e >= 0) {
            const TW* gr = wgu + (static_cast<size_t>(e) * 2 * ff + f) * W;
            float g, u;
            moe_dot2(gr, gr + static_cast<size_t>(ff) * W, xs, W, lane, vec, g, u);
            out = wt * moe_activate(g, u, limit, alpha, shift);
        }
        if (lane == 0) act[static_cast<size_t>(pair) * ff + f] = from_f32<TO>(out);
    }
}

template <typename TA, typename TW>
__global__ void moe_down_sparse_kernel(const TA* __restrict__ act, const TW* __restrict__ wd,
                                       const int32_t* __restrict__ ids, float* __restrict__ out, int W, int ff, int top,
                                       int E, int vec) {
    pdl_begin();
    extern __shared__ __align__(16) float as[];        // [top * ff]
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int i = threadIdx.x; i < top * ff; i += blockDim.x) as[i] = to_f32(act[static_cast<size_t>(t) * top * ff + i]);
    __syncthreads();
    const int n0 = blockIdx.y * MOE_SPARSE_FEATURES;
    for (int n = n0 + warp; n < min(W, n0 + MOE_SPARSE_FEATURES); n += MOE_SPARSE_WARPS) {
        const TW* row = wd + static_cast<size_t>(n) * E * ff;
        float acc = 0.0f;
        for (int k = 0; k < top; ++k) {
            const int e = ids[t * top + k];
            if (e >= 0) acc += moe_dot(row + static_cast<size_t>(e) * ff, as + k * ff, ff, lane, vec);
        }
        if (lane == 0) out[static_cast<size_t>(t) * W + n] = acc;
    }
}

extern "C" int llm_moe_sparse(const void* x, int x_dtype, const void* wgu, const void* wd, int w_dtype, const int32_t* ids,
                              const float* weights, void* act, float* out, int num_tokens, int W, int ff, int E, int top,
                              float limit, float alpha, float shift, uintptr_t stream) {
    if (num_tokens <= 0) return LLM_OK;
    if (W <= 0 || ff <= 0 || E <= 0 || top <= 0 || !(limit > 0.0f)) return LLM_REFUSED_SIZE;
    const size_t smem_a = static_cast<size_t>(W) * sizeof(float), smem_b = static_cast<size_t>(top) * ff * sizeof(float);
    if (smem_a > 48 * 1024 || smem_b > 48 * 1024) return LLM_REFUSED_SIZE;
    if (x_dtype != w_dtype) return LLM_REFUSED_DTYPE;       // the activations between the two kernels take the tokens' dtype
    const int vec = W % 8 == 0 && ff % 8 == 0 && aligned16(wgu) && aligned16(wd);
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    const dim3 grid_a(num_tokens * top, (ff + MOE_SPARSE_FEATURES - 1) / MOE_SPARSE_FEATURES);
    const dim3 grid_b(num_tokens, (W + MOE_SPARSE_FEATURES - 1) / MOE_SPARSE_FEATURES);
    const dim3 block(MOE_SPARSE_WARPS * 32);
    if (x_dtype == LLM_DT_F32) {
        launch_pdl((moe_gate_up_sparse_kernel<float, float, float>), grid_a, block, smem_a, s, static_cast<const float*>(x),
                   static_cast<const float*>(wgu), ids, weights, static_cast<float*>(act), W, ff, top, limit, alpha, vec, shift);
        launch_pdl((moe_down_sparse_kernel<float, float>), grid_b, block, smem_b, s, static_cast<const float*>(act),
                   static_cast<const float*>(wd), ids, out, W, ff, top, E, vec);
    } else if (x_dtype == LLM_DT_BF16) {
        launch_pdl((moe_gate_up_sparse_kernel<bf16, bf16, bf16>), grid_a, block, smem_a, s, static_cast<const bf16*>(x),
                   static_cast<const bf16*>(wgu), ids, weights, static_cast<bf16*>(act), W, ff, top, limit, alpha, vec, shift);
        launch_pdl((moe_down_sparse_kernel<bf16, bf16>), grid_b, block, smem_b, s, static_cast<const bf16*>(act),
                   static_cast<const bf16*>(wd), ids, out, W, ff, top, E, vec);
    } else {
        return LLM_REFUSED_DTYPE;
    }
    return launch_status();
}

// ---- prompt portions: tokens sorted by expert around the library's grouped matrix product -------------------
// moe_sort_kernel      (one block) counts the (token, choice) pairs of each expert, lays the experts' rows one
//                      after another and gives every pair its row: offs[e] = end of expert e's rows, pos[pair] =
//                      the pair's row, row_pair[row] = the pair (token = pair / top).  Which of an expert's
//                      rows a pair gets is not fixed; no result depends on it (a row's products are its own).
// moe_gather_kernel    xs[row] = x[token of the row]
// moe_act_pairs_kernel act[row, f] = w * g * sigmoid(alpha g) * (u + 1) from the grouped product's [rows, 2 ff]
// moe_combine_kernel   out[token] = sum over its choices of y[pos[pair]], in 32-bit, in the order of the choices
__global__ void moe_sort_kernel(const int32_t* __restrict__ ids, int pairs, int E, int32_t* __restrict__ offs,
                                int32_t* __restrict__ pos, int32_t* __restrict__ row_pair) {
    pdl_begin();
    extern __shared__ int sort_smem[];
    int* hist = sort_smem;            // [E]
    int* base = hist + E;             // [E]
    for (int e = threadIdx.x; e < E; e += blockDim.x) hist[e] = 0;
    __syncthreads();
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
        const int e = ids[p];
        if (e >= 0 && e < E) atomicAdd(&hist[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (int e = 0; e < E; ++e) {
            base[e] = run;
            run += hist[e];
            offs[e] = run;
            hist[e] = 0;              // becomes the cursor
        }
    }
    __syncthreads();
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
        const int e = ids[p];
        if (e >= 0 && e < E) {
            const int r = base[e] + atomicAdd(&hist[e], 1);
            pos[p] = r;
            row_pair[r] = p;
        } else {
            pos[p] = -1;
        }
    }
}

template <typename T>
__global__ void moe_gather_kernel(const T* __restrict__ x, const int32_t* __restrict__ row_pair, T* __restrict__ xs,
                                  int W, int top, int vec) {
    pdl_begin();
    const long long r = blockIdx.x;
    const T* src = x + static_cast<size_t>(row_pair[r] / top) * W;
    T* dst = xs + r * W;
    if (vec) {
        constexpr int PER = 16 / sizeof(T);
        for (int i = threadIdx.x * PER; i < W; i += blockDim.x * PER)
            *reinterpret_cast<uint4*>(dst + i) = *reinterpret_cast<const uint4*>(src + i);
    } else {
        for (int i = threadIdx.x; i < W; i += blockDim.x) dst[i] = src[i];
    }
}

template <typename T>
__global__ void moe_act_pairs_kernel(const T* __restrict__ gu, const int32_t* __restrict__ row_pair,
                                     const float* __restrict__ weights, T* __restrict__ act, int ff, float limit,
                                     float alpha, int vec, float shift) {
    pdl_begin();
    const long long r = blockIdx.x;
    const float w = weights[row_pair[r]];
    const T* g = gu + r * 2 * ff;
    T* o = act + r * ff;
    if (vec) {
        for (int f = (blockIdx.y * blockDim.x + threadIdx.x) * 8; f < ff; f += gridDim.y * blockDim.x * 8) {
            float a[8], b[8];
            load8(g + f, a);
            load8(g + ff + f, b);
#pragma unroll
            for (int c = 0; c < 8; ++c) a[c] = w * moe_activate(a[c], b[c], limit, alpha, shift);
            store8(o + f, a);
        }
    } else {
        for (int f = blockIdx.y * blockDim.x + threadIdx.x; f < ff; f += gridDim.y * blockDim.x) {
            o[f] = from_f32<T>(w * moe_activate(to_f32(g[f]), to_f32(g[ff + f]), limit, alpha, shift));
        }
    }
}

template <typename T>
__global__ void moe_combine_kernel(const T* __restrict__ y, const int32_t* __restrict__ pos, float* __restrict__ out,
                                   int W, int top, int vec) {
    pdl_begin();
    const long long t = blockIdx.x;
    if (vec) {
        for (int i = (blockIdx.y * blockDim.x + threadIdx.x) * 8; i < W; i += gridDim.y * blockDim.x * 8) {
            float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            for (int k = 0; k < top; ++k) {
                const int r = pos[t * top + k];
                if (r < 0) continue;
                float a[8];
                load8(y + static_cast<size_t>(r) * W + i, a);
#pragma unroll
                for (int c = 0; c < 8; ++c) acc[c] += a[c];
            }
            store8(out + t * W + i, acc);
        }
    } else {
        for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < W; i += gridDim.y * blockDim.x) {
            float acc = 0.0f;
            for (int k = 0; k < top; ++k) {
                const int r = pos[t * top + k];
                if (r >= 0) acc += to_f32(y[static_cast<size_t>(r) * W + i]);
            }
            out[t * W + i] = acc;
        }
    }
}

extern "C" int llm_moe_sort(const int32_t* ids, int pairs, int E, int32_t* offs, int32_t* pos, int32_t* row_pair,
                            uintptr_t stream) {
    if (pairs <= 0) return LLM_OK;
    if (E <= 0 || E > 4096) return LLM_REFUSED_SIZE;
    launch_pdl(moe_sort_kernel, dim3(1), dim3(1024), 2 * E * sizeof(int), reinterpret_cast<cudaStream_t>(stream), ids, pairs,
               E, offs, pos, row_pair);
    return launch_status();
}

// which = 0: gather (a = x [T, W], out = xs [pairs, W]); 1: activation (a = gu [pairs, 2 n], out = act [pairs, n]);
// 2: combine (a = y [pairs, n], out = float32 [T, n], index = pos).  n is the row width of `out`.
extern "C" int llm_moe_rows(int which, const void* a, int dtype, const int32_t* index, const float* weights, void* out,
                            int rows, int n, int top, float limit, float alpha, float shift, uintptr_t stream) {
    if (rows <= 0) return LLM_OK;
    if (n <= 0 || top <= 0 || which < 0 || which > 2) return LLM_REFUSED_SIZE;
    const int esz = dtype == LLM_DT_F32 ? 4 : 2;
    const int vec = (n % 8 == 0) && aligned16(a) && aligned16(out) && (static_cast<long long>(n) * esz) % 16 == 0;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    const int gy = which == 0 ? 1 : (n + 128 * 8 - 1) / (128 * 8);
    const dim3 grid(rows, gy), block(128);
    if (which == 0) {
        if (dtype == LLM_DT_F32) launch_pdl((moe_gather_kernel<float>), grid, block, 0, s, static_cast<const float*>(a), index,
                                            static_cast<float*>(out), n, top, vec);
        else if (dtype == LLM_DT_BF16) launch_pdl((moe_gather_kernel<bf16>), grid, block, 0, s, static_cast<const bf16*>(a), index,
                                                  static_cast<bf16*>(out), n, top, vec);
        else return LLM_REFUSED_DTYPE;
    } else if (which == 1) {
        if (dtype == LLM_DT_F32) launch_pdl((moe_act_pairs_kernel<float>), grid, block, 0, s, static_cast<const float*>(a), index,
                                            weights, static_cast<float*>(out), n, limit, alpha, vec, shift);
        else if (dtype == LLM_DT_BF16) launch_pdl((moe_act_pairs_kernel<bf16>), grid, block, 0, s, static_cast<const bf16*>(a),
                                                  index, weights, static_cast<bf16*>(out), n, limit, alpha, vec, shift);
        else return LLM_REFUSED_DTYPE;
    } else {
        if (dtype == LLM_DT_F32) launch_pdl((moe_combine_kernel<float>), grid, block, 0, s, static_cast<const float*>(a), index,
                                            static_cast<float*>(out), n, top, vec);
        else if (dtype == LLM_DT_BF16) launch_pdl((moe_combine_kernel<bf16>), grid, block, 0, s, static_cast<const bf16*>(a), index,
                                                  static_cast<float*>(out), n, top, vec);
        else return LLM_REFUSED_DTYPE;
    }
    return launch_status();
}

// What a routed feed-forward adds beside its experts' weighted sum: out[t] += idw[t] * x[t] (the share of a token's
// own input, for models whose router may pick "no expert") + shared[t] (an expert that every token runs), in 32-bit.
// `shared` may come as the `parts` k-splits of a product, `part_stride` floats apart.
template <typename TX>
__global__ void moe_finish_kernel(float* __restrict__ out, const TX* __restrict__ x, const float* __restrict__ idw,
                                  const float* __restrict__ shared, int parts, long long part_stride, long long total, int W) {
    pdl_begin();
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        float v = out[i];
        if (idw) v += idw[i / W] * to_f32(x[i]);
        if (shared)
            for (int k = 0; k < parts; ++k) v += shared[k * part_stride + i];
        out[i] = v;
    }
}

extern "C" int llm_moe_finish(float* out, const void* x, int x_dtype, const float* idw, const float* shared, int parts,
                              long long part_stride, int num_tokens, int W, uintptr_t stream) {
    if (num_tokens <= 0) return LLM_OK;
    if (W <= 0 || (idw && !x)) return LLM_REFUSED_SIZE;
    const long long total = static_cast<long long>(num_tokens) * W;
    const int threads = 256;
    const long long want = (total + threads - 1) / threads;
    const dim3 grid(static_cast<unsigned>(want < 4096 ? want : 4096));
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    if (parts < 1) parts = 1;
    if (x_dtype == LLM_DT_F32)
        launch_pdl((moe_finish_kernel<float>), grid, dim3(threads), 0, s, out, static_cast<const float*>(x), idw, shared, parts,
                   part_stride, total, W);
    else if (x_dtype == LLM_DT_BF16)
        launch_pdl((moe_finish_kernel<bf16>), grid, dim3(threads), 0, s, out, static_cast<const bf16*>(x), idw, shared, parts,
                   part_stride, total, W);
    else
        return LLM_REFUSED_DTYPE;
    return launch_status();
}
