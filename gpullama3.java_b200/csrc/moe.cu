// A routed feed-forward (mixture of experts): the router, and the experts for steps of few tokens.
//
//   moe_route     per token: logits z = W_r h (32-bit sums, W_r kept in 32 bits), scores s = softmax(z) over all experts.
//                 The experts form `n_groups` equal groups of neighbours; a group's score is its best expert's score, and
//                 only experts of the `keep_groups` best groups may be chosen.  The `top` allowed experts with the
//                 largest scores are chosen (ties: the lower index); their weights are their scores over the sum of
//                 the chosen scores (+ norm_eps).  A warp per token.
//   moe_expert_up / moe_expert_down
//                 the experts of every (token, chosen expert) pair as two weight-streaming kernels: a pair's gate and up
//                 rows meet the token's input, the gated epilogue follows (the same codes as the products' gated
//                 epilogues), and the down rows of a token's chosen experts meet its pairs' results, weighted and summed
//                 in the order of choice into the 32-bit residual stream.  Which expert a pair uses is read on the device,
//                 so a decode step's launches do not depend on the routing.
//   moe_group / moe_gather / moe_combine
//                 for prompts: the pairs are ordered by expert (counting sort; the order inside an expert's run does not
//                 change any result, a row of a product depends on its own input row only), the inputs gathered into that
//                 order, so that each expert's rows are one dense product for the tensor-core kernels, and the results
//                 carried back, weighted, into the residual stream.
#include "common.cuh"

namespace b200 {

constexpr int kMaxExperts = 1024;
constexpr int kMaxTop = 32;

template <typename T> struct Piece;  // 16 bytes of storage type T as floats
template <> struct Piece<float> {
    static constexpr int kElems = 4;
    __device__ static void load(const float* p, float* f) {
        const float4 v = *reinterpret_cast<const float4*>(p);
        f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
    }
};
template <> struct Piece<__nv_bfloat16> {
    static constexpr int kElems = 8;
    __device__ static void load(const __nv_bfloat16* p, float* f) {
        const uint4 v = *reinterpret_cast<const uint4*>(p);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            f[2 * i] = __uint_as_float(w[i] << 16);
            f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
};

// sum_k w[k] x[k] over a warp: lanes take 16-byte pieces of the weight row when VEC, single elements otherwise;
// x is in shared memory as floats
template <typename T, bool VEC>
__device__ __forceinline__ float warp_dot(const T* __restrict__ w, const float* __restrict__ x, int K, int lane) {
    float acc = 0.f;
    if (VEC) {
        constexpr int E = Piece<T>::kElems;
        for (int k = lane * E; k < K; k += 32 * E) {
            float f[E];
            Piece<T>::load(w + k, f);
#pragma unroll
            for (int e = 0; e < E; ++e) acc += f[e] * x[k + e];
        }
    } else {
        for (int k = lane; k < K; k += 32) acc += to_f32<T>(w[k]) * x[k];
    }
    return warp_sum(acc);
}

// ------------------------------------------------------------------------------------------------ router
struct RouteArgs {
    const void* h;          // [T][ld_h], the run's storage type
    int ld_h;
    const float* router;    // [n_experts][width]
    int* chosen;            // [T][top]
    float* weights;         // [T][top]
    float* scores;          // [T][n_experts] or null: the softmax scores, for inspection
    int n_tokens, width, n_experts, n_groups, keep_groups, top;
    float norm_eps;
};

constexpr int kRouteWarps = 4;

template <typename T>
__global__ void __launch_bounds__(kRouteWarps * 32)
moe_route_kernel(RouteArgs a) {
    extern __shared__ float smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float* x = smem + (size_t)warp * (a.width + a.n_experts + a.n_groups);   // the token's input
    float* s = x + a.width;                                                   // scores; chosen or barred ones turn negative
    float* gs = s + a.n_experts;                                              // group scores
    const int t = blockIdx.x * kRouteWarps + warp;
    if (t >= a.n_tokens) return;
    const T* hr = (const T*)a.h + (size_t)t * a.ld_h;
    for (int k = lane; k < a.width; k += 32) x[k] = to_f32<T>(hr[k]);
    __syncwarp();
    float m = -INFINITY;
    for (int e = 0; e < a.n_experts; ++e) {
        const float z = warp_dot<float, false>(a.router + (size_t)e * a.width, x, a.width, lane);
        if (lane == 0) s[e] = z;
        m = fmaxf(m, z);
    }
    __syncwarp();
    float sum = 0.f;
    for (int e = lane; e < a.n_experts; e += 32) sum += expf(s[e] - m);
    sum = warp_sum(sum);
    for (int e = lane; e < a.n_experts; e += 32) {
        s[e] = expf(s[e] - m) / sum;
        if (a.scores) a.scores[(size_t)t * a.n_experts + e] = s[e];
    }
    __syncwarp();
    // groups: keep the best `keep_groups`, bar the experts of the others
    const int per = a.n_experts / a.n_groups;
    if (a.keep_groups < a.n_groups) {
        for (int g = lane; g < a.n_groups; g += 32) {
            float best = -1.f;
            for (int i = 0; i < per; ++i) best = fmaxf(best, s[g * per + i]);
            gs[g] = best;
        }
        __syncwarp();
        for (int r = 0; r < a.keep_groups; ++r) {
            float bv = -2.f;
            int bi = 0x7fffffff;
            for (int g = lane; g < a.n_groups; g += 32)
                if (gs[g] > bv) { bv = gs[g]; bi = g; }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
                const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
            }
            if (lane == 0) gs[bi] = -3.f;    // taken
            __syncwarp();
        }
        for (int e = lane; e < a.n_experts; e += 32)
            if (gs[e / per] != -3.f) s[e] = -1.f - s[e];   // barred: negative, the score recoverable (never needed)
        __syncwarp();
    }
    // the `top` best allowed experts, one after the other
    float chosen_sum = 0.f;
    float my_w = 0.f;
    int my_e = 0;
    for (int r = 0; r < a.top; ++r) {
        float bv = -1.f;
        int bi = 0x7fffffff;
        for (int e = lane; e < a.n_experts; e += 32)
            if (s[e] > bv) { bv = s[e]; bi = e; }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        chosen_sum += bv;
        if (lane == r) { my_w = bv; my_e = bi; }
        if (lane == 0) s[bi] = -1.f;
        __syncwarp();
    }
    if (lane < a.top) {
        a.chosen[(size_t)t * a.top + lane] = my_e;
        a.weights[(size_t)t * a.top + lane] = my_w / (chosen_sum + a.norm_eps);
    }
}

// ------------------------------------------------------------------------------------------------ experts, pair by pair
__device__ __forceinline__ float gated_value(float gate, float up, int act, float limit, float slope) {
    if (act == 2) {
        const float g = fminf(gate, limit), u = fminf(fmaxf(up, -limit), limit);
        return g / (1.0f + expf(-slope * g)) * (u + 1.0f);
    }
    if (act == 1) return 0.5f * gate * (1.0f + tanhf(0.7978845608028654f * (gate + 0.044715f * gate * gate * gate))) * up;
    return gate / (1.0f + expf(-gate)) * up;
}

constexpr int kExpertWarps = 4;
constexpr int kUpPerWarp = 2;     // gate/up pairs a warp computes one after the other

// y[pair][j] = act(W_gu[e][2 j] . h[t], W_gu[e][2 j + 1] . h[t]);  grid (ceil(ff / (warps * kUpPerWarp)), pairs)
template <typename T, bool VEC>
__global__ void __launch_bounds__(kExpertWarps * 32)
moe_expert_up_kernel(const T* __restrict__ h, int ld_h, const T* __restrict__ w_gu, const int* __restrict__ chosen,
                     T* __restrict__ y, int width, int ff, int top, int act, float limit, float slope) {
    extern __shared__ float x[];
    const int pair = blockIdx.y, t = pair / top, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const T* hr = h + (size_t)t * ld_h;
    for (int k = threadIdx.x; k < width; k += blockDim.x) x[k] = to_f32<T>(hr[k]);
    __syncthreads();
    const int e = chosen[pair];
    const T* w = w_gu + (size_t)e * 2 * ff * width;
#pragma unroll
    for (int i = 0; i < kUpPerWarp; ++i) {
        const int j = (blockIdx.x * kExpertWarps + warp) * kUpPerWarp + i;
        if (j >= ff) break;
        const float gate = warp_dot<T, VEC>(w + (size_t)(2 * j) * width, x, width, lane);
        const float up = warp_dot<T, VEC>(w + (size_t)(2 * j + 1) * width, x, width, lane);
        if (lane == 0) y[(size_t)pair * ff + j] = from_f32<T>(gated_value(gate, up, act, limit, slope));
    }
}

constexpr int kDownPerWarp = 2;

// residual[t][c] += sum_k weights[t][k] (W_down[e_k][c] . y[t top + k]);  grid (ceil(width / (warps * kDownPerWarp)), T)
template <typename T, bool VEC>
__global__ void __launch_bounds__(kExpertWarps * 32)
moe_expert_down_kernel(const T* __restrict__ y, const T* __restrict__ w_down, const int* __restrict__ chosen,
                       const float* __restrict__ weights, float* __restrict__ residual, int width, int ff, int top) {
    extern __shared__ float ys[];          // [top][ff]
    __shared__ int e_s[kMaxTop];
    __shared__ float w_s[kMaxTop];
    const int t = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int i = threadIdx.x; i < top * ff; i += blockDim.x) ys[i] = to_f32<T>(y[(size_t)t * top * ff + i]);
    if (threadIdx.x < top) {
        e_s[threadIdx.x] = chosen[(size_t)t * top + threadIdx.x];
        w_s[threadIdx.x] = weights[(size_t)t * top + threadIdx.x];
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < kDownPerWarp; ++i) {
        const int c = (blockIdx.x * kExpertWarps + warp) * kDownPerWarp + i;
        if (c >= width) break;
        float total = 0.f;
        for (int k = 0; k < top; ++k) {
            const T* w = w_down + ((size_t)e_s[k] * width + c) * ff;
            total += w_s[k] * warp_dot<T, VEC>(w, ys + (size_t)k * ff, ff, lane);
        }
        if (lane == 0) residual[(size_t)t * width + c] += total;
    }
}

// ------------------------------------------------------------------------------------------------ prompts: order by expert
// One CTA.  offsets[e] .. offsets[e + 1]: the run of expert e among the ordered pairs; order[p]: which pair stands at
// place p; place[pair]: where a pair stands.
__global__ void __launch_bounds__(1024)
moe_group_kernel(const int* __restrict__ chosen, int n_pairs, int n_experts, int* __restrict__ offsets,
                 int* __restrict__ order, int* __restrict__ place) {
    __shared__ int count[kMaxExperts + 1];
    for (int e = threadIdx.x; e <= n_experts; e += blockDim.x) count[e] = 0;
    __syncthreads();
    for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) atomicAdd(&count[chosen[p]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (int e = 0; e < n_experts; ++e) {
            const int n = count[e];
            offsets[e] = run;
            count[e] = run;      // from here on: the next free place of the expert's run
            run += n;
        }
        offsets[n_experts] = run;
    }
    __syncthreads();
    for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
        const int at = atomicAdd(&count[chosen[p]], 1);
        order[at] = p;
        place[p] = at;
    }
}

// x_sorted[p] = h[order[p] / top]
template <typename T>
__global__ void moe_gather_kernel(const T* __restrict__ h, int ld_h, const int* __restrict__ order, T* __restrict__ out,
                                  int width, int top) {
    const int p = blockIdx.x;
    const T* src = h + (size_t)(order[p] / top) * ld_h;
    T* dst = out + (size_t)p * width;
    for (int k = threadIdx.x; k < width; k += blockDim.x) dst[k] = src[k];
}

// residual[t] += sum_k weights[t][k] o[place[t top + k]], in the order of choice
__global__ void moe_combine_kernel(const float* __restrict__ o, const int* __restrict__ place, const float* __restrict__ weights,
                                   float* __restrict__ residual, int width, int top) {
    const int t = blockIdx.x;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        float total = 0.f;
        for (int k = 0; k < top; ++k)
            total += weights[(size_t)t * top + k] * o[(size_t)place[(size_t)t * top + k] * width + c];
        residual[(size_t)t * width + c] += total;
    }
}

}  // namespace b200

extern "C" int b200_moe_route(const void* h, int ld_h, int dtype, const float* router, int* chosen, float* weights,
                              float* scores, int n_tokens, int width, int n_experts, int n_groups, int keep_groups, int top,
                              float norm_eps, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (n_experts < 1 || n_experts > b200::kMaxExperts || top < 1 || top > 32 || top > n_experts || n_groups < 1 ||
        n_experts % n_groups || keep_groups < 1 || keep_groups > n_groups || top > keep_groups * (n_experts / n_groups))
        return b200::kErrBadArgument;
    const size_t smem = sizeof(float) * b200::kRouteWarps * ((size_t)width + n_experts + n_groups);
    if (smem > 200 * 1024) return b200::kErrUnsupportedSize;
    const b200::RouteArgs a = {h, ld_h, router, chosen, weights, scores, n_tokens, width, n_experts, n_groups, keep_groups, top, norm_eps};
    B200_DISPATCH_DTYPE(dtype, T,
        auto kernel = b200::moe_route_kernel<T>;
        if (smem > 48 * 1024) {
            const int e = (int)cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != 0) return e;
        }
        kernel<<<(n_tokens + b200::kRouteWarps - 1) / b200::kRouteWarps, b200::kRouteWarps * 32, smem, stream>>>(a));
    return b200::launch_status();
}

// h [T][ld_h]; w_gu [n_experts][2 ff][width] (gate and up rows interleaved); w_down [n_experts][width][ff];
// y [T top][ff] scratch of the run's type; residual [T][width] 32-bit.  act: 0 SiLU, 1 GELU (tanh form), 2 clamped.
extern "C" int b200_moe_experts(const void* h, int ld_h, int dtype, const void* w_gu, const void* w_down, const int* chosen,
                                const float* weights, void* y, float* residual, int n_tokens, int width, int ff, int top,
                                int act, float limit, float slope, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (top < 1 || top > b200::kMaxTop || width < 1 || ff < 1 || act < 0 || act > 2) return b200::kErrBadArgument;
    const long long pairs = (long long)n_tokens * top;
    if (pairs > 65535 || n_tokens > 65535) return b200::kErrUnsupportedSize;
    const size_t smem_up = sizeof(float) * width, smem_down = sizeof(float) * (size_t)top * ff;
    if (smem_up > 200 * 1024 || smem_down > 200 * 1024) return b200::kErrUnsupportedSize;
    const int el = dtype == b200::kF32 ? 4 : 8;
    const bool vec = width % el == 0 && ff % el == 0 && ld_h % el == 0 &&
                     ((((uintptr_t)w_gu) | ((uintptr_t)w_down)) & 15) == 0;
    const dim3 grid_up((ff + b200::kExpertWarps * b200::kUpPerWarp - 1) / (b200::kExpertWarps * b200::kUpPerWarp), (unsigned)pairs);
    const dim3 grid_down((width + b200::kExpertWarps * b200::kDownPerWarp - 1) / (b200::kExpertWarps * b200::kDownPerWarp), n_tokens);
#define B200_MOE_GO(T, VEC)                                                                                                  \
    do {                                                                                                                     \
        auto up = b200::moe_expert_up_kernel<T, VEC>;                                                                        \
        auto down = b200::moe_expert_down_kernel<T, VEC>;                                                                    \
        if (smem_up > 48 * 1024) cudaFuncSetAttribute(up, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_up);        \
        if (smem_down > 48 * 1024) cudaFuncSetAttribute(down, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_down);  \
        up<<<grid_up, b200::kExpertWarps * 32, smem_up, stream>>>((const T*)h, ld_h, (const T*)w_gu, chosen, (T*)y, width, ff, \
                                                                  top, act, limit, slope);                                   \
        down<<<grid_down, b200::kExpertWarps * 32, smem_down, stream>>>((const T*)y, (const T*)w_down, chosen, weights,      \
                                                                        residual, width, ff, top);                           \
    } while (0)
    B200_DISPATCH_DTYPE(dtype, T, if (vec) B200_MOE_GO(T, true); else B200_MOE_GO(T, false));
#undef B200_MOE_GO
    return b200::launch_status();
}

extern "C" int b200_moe_group(const int* chosen, int n_pairs, int n_experts, int* offsets, int* order, int* place,
                              cudaStream_t stream) {
    if (n_pairs <= 0) return 0;
    if (n_experts < 1 || n_experts > b200::kMaxExperts) return b200::kErrBadArgument;
    b200::moe_group_kernel<<<1, 1024, 0, stream>>>(chosen, n_pairs, n_experts, offsets, order, place);
    return b200::launch_status();
}

extern "C" int b200_moe_gather(const void* h, int ld_h, int dtype, const int* order, void* out, int n_pairs, int width,
                               int top, cudaStream_t stream) {
    if (n_pairs <= 0) return 0;
    B200_DISPATCH_DTYPE(dtype, T,
        b200::moe_gather_kernel<T><<<n_pairs, 128, 0, stream>>>((const T*)h, ld_h, order, (T*)out, width, top));
    return b200::launch_status();
}

extern "C" int b200_moe_combine(const float* o, const int* place, const float* weights, float* residual, int n_tokens,
                                int width, int top, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    b200::moe_combine_kernel<<<n_tokens, 256, 0, stream>>>(o, place, weights, residual, width, top);
    return b200::launch_status();
}
