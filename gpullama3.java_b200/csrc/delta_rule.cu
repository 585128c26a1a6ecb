// The gated delta rule with one decay per key channel, and the short causal convolution in front of it.
//
// Per sequence and head the mixer keeps a matrix S [d_k, d_v] of 32-bit numbers.  A token with unit-length
// query q and key k [d_k], value v [d_v], write strength beta and per-channel decay g [d_k] in (0, 1) does
//     S <- diag(g) S ;  u = beta (v - S^T k) ;  S <- S + k u^T ;  o = S^T q
// in this order.  Column j of S only ever meets column j of v, u and o, so the columns are independent chains:
// a thread holds RPT rows of one column in registers, R neighbouring lanes share a column (d_k <= R * RPT, rows
// beyond d_k are zero and stay zero), and the two dot products of a token are finished by log2(R) exchanges.
// Tokens are taken in chunks of kChunk: the CTA first prepares the chunk in shared memory (unit norms of q and k
// from the convolution's output, the query scale, beta = sigmoid(.), g = exp(-exp(A_log) softplus(a + dt_bias)),
// all 32-bit) and then walks it.  The same kernel serves a prompt, a portion of one and a single decoded token: a
// sequence's tokens are rows cu_seqlens[i] .. cu_seqlens[i + 1] of the step, its state sits in its cache slot.
//
// The convolution: channel c of token t gets sum_j w[c, j] x[t - (taps - 1) + j, c] followed by SiLU, where inputs
// before the step's first token come from the slot's state (the last taps - 1 inputs of the sequence, zero at its
// start); conv_state_update then stores the step's last taps - 1 inputs there.
#include "common.cuh"

namespace b200 {

constexpr int kScanThreads = 128;
constexpr int kChunk = 16;
constexpr int kMaxTaps = 16;

template <typename T>
__global__ void causal_conv_silu_kernel(const T* __restrict__ x, int ld_x, const float* __restrict__ w,
                                        const float* __restrict__ state, size_t slot_stride, const int* __restrict__ slots,
                                        const int* __restrict__ seq_ids, const int* __restrict__ cu_seqlens,
                                        T* __restrict__ out, int ld_out, int channels, int taps) {
    const int t = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= channels) return;
    const int seq = seq_ids[t];
    const int local = t - cu_seqlens[seq];
    const float* st = state + (size_t)slots[seq] * slot_stride;   // [taps - 1][channels], oldest first
    float acc = 0.f;
    for (int j = 0; j < taps; ++j) {
        const int back = taps - 1 - j;          // how many tokens before t
        float v;
        if (local - back >= 0) v = to_f32<T>(x[(size_t)(t - back) * ld_x + c]);
        else v = st[(size_t)(taps - 1 + local - back) * channels + c];
        acc += w[(size_t)c * taps + j] * v;
    }
    out[(size_t)t * ld_out + c] = from_f32<T>(acc / (1.0f + expf(-acc)));
}

template <typename T>
__global__ void conv_state_update_kernel(const T* __restrict__ x, int ld_x, float* __restrict__ state, size_t slot_stride,
                                         const int* __restrict__ slots, const int* __restrict__ cu_seqlens, int channels,
                                         int taps) {
    const int seq = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= channels) return;
    const int first = cu_seqlens[seq], n = cu_seqlens[seq + 1] - first;
    float* st = state + (size_t)slots[seq] * slot_stride;
    float fresh[kMaxTaps];
#pragma unroll
    for (int m = 0; m < kMaxTaps; ++m) {
        if (m >= taps - 1) break;
        const int idx = n - (taps - 1) + m;     // among the step's tokens; negative: still an older input
        fresh[m] = idx >= 0 ? to_f32<T>(x[(size_t)(first + idx) * ld_x + c]) : st[(size_t)(m + n) * channels + c];
    }
#pragma unroll
    for (int m = 0; m < kMaxTaps; ++m) {
        if (m >= taps - 1) break;
        st[(size_t)m * channels + c] = fresh[m];
    }
}

struct ScanArgs {
    const void* qkv;        // [T, ld_qkv]: convolved q [kv_heads d_k], k [kv_heads d_k], v [heads d_v]
    int ld_qkv;
    const void* beta;       // [T, ld_beta], column h: before the sigmoid
    int ld_beta;
    const void* decay;      // [T, ld_decay], column h d_k + i: before dt_bias and softplus
    int ld_decay;
    const float* dt_bias;   // [heads d_k]
    const float* a_log;     // [heads]
    float* state;           // per slot: [heads][d_k][d_v]
    size_t slot_stride;
    const int* slots;
    const int* cu_seqlens;
    float* out;             // [T, heads d_v] 32-bit
    int heads, kv_heads, d_k, d_v, lanes;   // lanes = R
    float q_scale, unit_eps;
};

__device__ __forceinline__ float softplus(float x) { return x > 20.f ? x : log1pf(expf(x)); }

template <typename T, int RPT>
__global__ void __launch_bounds__(kScanThreads)
delta_rule_scan_kernel(ScanArgs a) {
    extern __shared__ float smem[];
    const int R = a.lanes, dpad = R * RPT, cols = kScanThreads / R;
    float* q_s = smem;                       // [kChunk][dpad]
    float* k_s = q_s + kChunk * dpad;
    float* g_s = k_s + kChunk * dpad;
    float* v_s = g_s + kChunk * dpad;        // [kChunk][cols]
    float* b_s = v_s + kChunk * cols;        // [kChunk]

    const int h = blockIdx.y, seq = blockIdx.z, col0 = blockIdx.x * cols;
    const int kvh = h / (a.heads / a.kv_heads);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int col = col0 + tid / R, r = tid % R;
    const bool live = col < a.d_v;
    const int first = a.cu_seqlens[seq], n = a.cu_seqlens[seq + 1] - first;
    float* S_g = a.state + (size_t)a.slots[seq] * a.slot_stride + (size_t)h * a.d_k * a.d_v;
    const T* qkv = (const T*)a.qkv;
    const T* beta = (const T*)a.beta;
    const T* decay = (const T*)a.decay;
    const float neg_rate = -expf(a.a_log[h]);
    const int k_off = a.kv_heads * a.d_k, v_off = 2 * a.kv_heads * a.d_k;

    float S[RPT];
#pragma unroll
    for (int i = 0; i < RPT; ++i) {
        const int row = r * RPT + i;
        S[i] = (live && row < a.d_k) ? S_g[(size_t)row * a.d_v + col] : 0.f;
    }

    for (int base = 0; base < n; base += kChunk) {
        const int m = min(kChunk, n - base);
        __syncthreads();   // the chunk before has been walked
        for (int tt = warp; tt < m; tt += kScanThreads / 32) {
            const size_t t = (size_t)first + base + tt;
            const T* qr = qkv + t * a.ld_qkv + (size_t)kvh * a.d_k;
            const T* kr = qr + k_off;
            float sq = 0.f, sk = 0.f;
            for (int i = lane; i < a.d_k; i += 32) {
                const float qv = to_f32<T>(qr[i]), kv = to_f32<T>(kr[i]);
                sq += qv * qv;
                sk += kv * kv;
            }
            sq = warp_sum(sq);
            sk = warp_sum(sk);
            const float fq = a.q_scale / sqrtf(sq + a.unit_eps), fk = 1.0f / sqrtf(sk + a.unit_eps);
            const T* dr = decay + t * a.ld_decay + (size_t)h * a.d_k;
            for (int i = lane; i < dpad; i += 32) {
                float qv = 0.f, kv = 0.f, gv = 1.f;
                if (i < a.d_k) {
                    qv = to_f32<T>(qr[i]) * fq;
                    kv = to_f32<T>(kr[i]) * fk;
                    gv = expf(neg_rate * softplus(to_f32<T>(dr[i]) + a.dt_bias[(size_t)h * a.d_k + i]));
                }
                q_s[tt * dpad + i] = qv;
                k_s[tt * dpad + i] = kv;
                g_s[tt * dpad + i] = gv;
            }
            const T* vr = qkv + t * a.ld_qkv + v_off + (size_t)h * a.d_v + col0;
            for (int c = lane; c < cols; c += 32) v_s[tt * cols + c] = (col0 + c < a.d_v) ? to_f32<T>(vr[c]) : 0.f;
            if (lane == 0) b_s[tt] = 1.0f / (1.0f + expf(-to_f32<T>(beta[t * a.ld_beta + h])));
        }
        __syncthreads();
        for (int tt = 0; tt < m; ++tt) {
            const float* qp = q_s + tt * dpad + r * RPT;
            const float* kp = k_s + tt * dpad + r * RPT;
            const float* gp = g_s + tt * dpad + r * RPT;
            float dot = 0.f;
#pragma unroll
            for (int i = 0; i < RPT; ++i) {
                S[i] *= gp[i];
                dot += S[i] * kp[i];
            }
            for (int o = R >> 1; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
            const float u = b_s[tt] * (v_s[tt * cols + tid / R] - dot);
            float outv = 0.f;
#pragma unroll
            for (int i = 0; i < RPT; ++i) {
                S[i] += kp[i] * u;
                outv += S[i] * qp[i];
            }
            for (int o = R >> 1; o > 0; o >>= 1) outv += __shfl_xor_sync(0xffffffffu, outv, o);
            if (live && r == 0) a.out[((size_t)first + base + tt) * a.heads * a.d_v + (size_t)h * a.d_v + col] = outv;
        }
    }
#pragma unroll
    for (int i = 0; i < RPT; ++i) {
        const int row = r * RPT + i;
        if (live && row < a.d_k) S_g[(size_t)row * a.d_v + col] = S[i];
    }
}

template <typename T, int RPT>
static int launch_scan(const ScanArgs& a, int n_seqs, cudaStream_t stream) {
    const int cols = kScanThreads / a.lanes, dpad = a.lanes * RPT;
    const size_t smem = sizeof(float) * ((size_t)kChunk * (3 * dpad + cols + 1));
    auto kernel = delta_rule_scan_kernel<T, RPT>;
    if (smem > 48 * 1024) {
        const int e = (int)cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != 0) return e;
    }
    dim3 grid((a.d_v + cols - 1) / cols, a.heads, n_seqs);
    kernel<<<grid, kScanThreads, smem, stream>>>(a);
    return launch_status();
}

}  // namespace b200

extern "C" int b200_causal_conv_silu(const void* x, int ld_x, const float* w, float* state, long long slot_stride,
                                     const int* slots, const int* seq_ids, const int* cu_seqlens, void* out, int ld_out,
                                     int dtype, int n_tokens, int n_seqs, int channels, int taps, int update_state,
                                     cudaStream_t stream) {
    if (n_tokens <= 0 || channels <= 0) return 0;
    if (taps < 1 || taps > b200::kMaxTaps) return b200::kErrUnsupportedSize;
    if (n_tokens > 65535 || n_seqs > 65535) return b200::kErrUnsupportedSize;
    dim3 grid((channels + 127) / 128, n_tokens), grid_u((channels + 127) / 128, n_seqs);
    B200_DISPATCH_DTYPE(dtype, T,
        b200::causal_conv_silu_kernel<T><<<grid, 128, 0, stream>>>((const T*)x, ld_x, w, state, (size_t)slot_stride, slots,
                                                                   seq_ids, cu_seqlens, (T*)out, ld_out, channels, taps);
        if (update_state && taps > 1)
            b200::conv_state_update_kernel<T><<<grid_u, 128, 0, stream>>>((const T*)x, ld_x, state, (size_t)slot_stride, slots,
                                                                          cu_seqlens, channels, taps));
    return b200::launch_status();
}

// The rows a thread holds (rows_per_thread: 8, 12, 16, 24 or 32) times the lanes that share a column (a power of two up
// to 16) must cover d_k; b200_delta_rule_plan picks the pair for a d_k (0 when none fits).
extern "C" int b200_delta_rule_plan(int d_k, int* rows_per_thread, int* lanes) {
    const int options[5] = {16, 24, 12, 32, 8};
    int best = 0, best_pad = 1 << 30;
    for (int oi = 0; oi < 5; ++oi)
        for (int R = 1; R <= 16; R *= 2) {
            const int pad = options[oi] * R;
            if (pad >= d_k && pad < best_pad) {
                best_pad = pad;
                best = options[oi];
                *rows_per_thread = options[oi];
                *lanes = R;
            }
        }
    return best;
}

extern "C" int b200_delta_rule_scan(const void* qkv, int ld_qkv, const void* beta, int ld_beta, const void* decay,
                                    int ld_decay, const float* dt_bias, const float* a_log, float* state,
                                    long long slot_stride, const int* slots, const int* cu_seqlens, float* out, int dtype,
                                    int n_seqs, int heads, int kv_heads, int d_k, int d_v, float q_scale, float unit_eps,
                                    cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (heads < 1 || kv_heads < 1 || heads % kv_heads || d_k < 1 || d_v < 1 || n_seqs > 65535 || heads > 65535)
        return b200::kErrBadArgument;
    int rpt = 0, lanes = 0;
    if (!b200_delta_rule_plan(d_k, &rpt, &lanes)) return b200::kErrUnsupportedSize;
    b200::ScanArgs a = {qkv, ld_qkv, beta, ld_beta, decay, ld_decay, dt_bias, a_log, state, (size_t)slot_stride, slots,
                        cu_seqlens, out, heads, kv_heads, d_k, d_v, lanes, q_scale, unit_eps};
#define B200_SCAN(RPT) B200_DISPATCH_DTYPE(dtype, T, return b200::launch_scan<T, RPT>(a, n_seqs, stream))
    switch (rpt) {
        case 8: B200_SCAN(8);
        case 12: B200_SCAN(12);
        case 16: B200_SCAN(16);
        case 24: B200_SCAN(24);
        case 32: B200_SCAN(32);
    }
#undef B200_SCAN
    return b200::kErrUnsupportedSize;
}
