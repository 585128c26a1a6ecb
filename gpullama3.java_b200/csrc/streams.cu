// Several residual streams side by side (hyper-connections).
//
// The residual stream of a token is S rows of `width` 32-bit numbers, [T, S, width].  A sublayer reads one
// weighted sum of the streams, and its result y goes back into every stream while the streams are mixed
// among themselves:
//     u      = sum_a  read[a] x_a                            (streams_read_norm: u is normalised at once)
//     x_j  <-  sum_a  mix[a, j] x_a  +  write[j] y           (streams_combine, in place, all j from the old x)
// streams_combine is also what opens the streams (S_in = 1, mix = ones: every stream starts as the embedding)
// and what closes them (S_out = 1, mix = ones: the model's output is their sum).  All sums are 32-bit.
#include "common.cuh"

namespace b200 {

constexpr int kMaxStreams = 8;
constexpr int kStreamThreads = 256;

// out[t, j, c] = sum_a mix[a * s_out + j] * x[t, a, c]  (+ write[j] * y[t, c]).  `out` may be `x` itself when
// s_in == s_out: a thread reads the s_in numbers of its (t, c) before it writes the s_out.
template <int VEC>
__global__ void __launch_bounds__(kStreamThreads)
streams_combine_kernel(const float* __restrict__ x, float* out, const float* __restrict__ mix,
                       const float* __restrict__ write, const float* __restrict__ y, int s_in, int s_out, int width,
                       size_t n_units) {   // units of VEC numbers: T * width / VEC
    __shared__ float m_s[kMaxStreams * kMaxStreams], w_s[kMaxStreams];
    for (int i = threadIdx.x; i < s_in * s_out; i += kStreamThreads) m_s[i] = mix[i];
    for (int i = threadIdx.x; i < s_out; i += kStreamThreads) w_s[i] = (write != nullptr) ? write[i] : 0.f;
    __syncthreads();
    const int wv = width / VEC;
    for (size_t u = (size_t)blockIdx.x * kStreamThreads + threadIdx.x; u < n_units; u += (size_t)gridDim.x * kStreamThreads) {
        const size_t t = u / wv;
        const int c = (int)(u % wv) * VEC;
        float in[kMaxStreams][VEC];
#pragma unroll
        for (int a = 0; a < kMaxStreams; ++a) {
            if (a >= s_in) break;
            const float* p = x + (t * s_in + a) * width + c;
            if (VEC == 4) {
                const float4 v = *reinterpret_cast<const float4*>(p);
                in[a][0] = v.x; in[a][1] = v.y; in[a][2] = v.z; in[a][3] = v.w;
            } else {
                in[a][0] = p[0];
            }
        }
        float yv[VEC];
#pragma unroll
        for (int e = 0; e < VEC; ++e) yv[e] = 0.f;
        if (y != nullptr) {
            const float* p = y + t * width + c;
            if (VEC == 4) {
                const float4 v = *reinterpret_cast<const float4*>(p);
                yv[0] = v.x; yv[1] = v.y; yv[2] = v.z; yv[3] = v.w;
            } else {
                yv[0] = p[0];
            }
        }
#pragma unroll
        for (int j = 0; j < kMaxStreams; ++j) {
            if (j >= s_out) break;
            float acc[VEC];
#pragma unroll
            for (int e = 0; e < VEC; ++e) acc[e] = 0.f;
#pragma unroll
            for (int a = 0; a < kMaxStreams; ++a) {
                if (a >= s_in) break;
                const float m = m_s[a * s_out + j];
#pragma unroll
                for (int e = 0; e < VEC; ++e) acc[e] += m * in[a][e];
            }
            if (y != nullptr) {
#pragma unroll
                for (int e = 0; e < VEC; ++e) acc[e] += w_s[j] * yv[e];
            }
            float* o = out + (t * s_out + j) * width + c;
            if (VEC == 4) *reinterpret_cast<float4*>(o) = make_float4(acc[0], acc[1], acc[2], acc[3]);
            else o[0] = acc[0];
        }
    }
}

// out[r] = w * u / sqrt(mean(u^2) + eps) with u = sum_a read[a] x[row(r), a, :]: the read of a sublayer and its
// norm in one pass.  `rows` (optional) selects tokens, as in rmsnorm.  A CTA per row; u stays in registers for
// widths up to kStreamKeep * 256 and is formed again from x beyond that.
constexpr int kStreamKeep = 8;

template <typename TO>
__global__ void __launch_bounds__(kStreamThreads)
streams_read_norm_kernel(const float* __restrict__ x, const float* __restrict__ read, const float* __restrict__ w,
                         TO* __restrict__ out, const int* __restrict__ rows, int n_streams, int width, float eps) {
    __shared__ float scratch[33];
    __shared__ float r_s[kMaxStreams];
    if (threadIdx.x < n_streams) r_s[threadIdx.x] = read[threadIdx.x];
    __syncthreads();
    const int r = blockIdx.x;
    const float* xr = x + (size_t)(rows ? rows[r] : r) * n_streams * width;
    float keep[kStreamKeep];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < kStreamKeep; ++k) {
        const int c = k * kStreamThreads + threadIdx.x;
        float u = 0.f;
        if (c < width)
            for (int a = 0; a < n_streams; ++a) u += r_s[a] * xr[(size_t)a * width + c];
        keep[k] = u;
        ss += u * u;
    }
    for (int c = kStreamKeep * kStreamThreads + threadIdx.x; c < width; c += kStreamThreads) {
        float u = 0.f;
        for (int a = 0; a < n_streams; ++a) u += r_s[a] * xr[(size_t)a * width + c];
        ss += u * u;
    }
    ss = block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)width + eps);
    TO* o = out + (size_t)r * width;
#pragma unroll
    for (int k = 0; k < kStreamKeep; ++k) {
        const int c = k * kStreamThreads + threadIdx.x;
        if (c < width) o[c] = from_f32<TO>(w[c] * (scale * keep[k]));
    }
    for (int c = kStreamKeep * kStreamThreads + threadIdx.x; c < width; c += kStreamThreads) {
        float u = 0.f;
        for (int a = 0; a < n_streams; ++a) u += r_s[a] * xr[(size_t)a * width + c];
        o[c] = from_f32<TO>(w[c] * (scale * u));
    }
}

// The write-back of one sublayer and the read of the next in one pass over a token's streams (a CTA per token):
//     x_j <- sum_a mix[a, j] x_a + write[j] y      (in place)
//     y   <- 0                                     (the next sublayer's last product adds into it again)
//     out  = w * u / sqrt(mean(u^2) + eps),  u = sum_j read[j] x_j     (only when `read` is given)
// so the new streams are not read again for the norm, and nothing else has to clear y.
template <int VEC> struct StreamVec;
template <> struct StreamVec<4> {
    __device__ static void load(const float* p, float (&f)[4]) {
        const float4 v = *reinterpret_cast<const float4*>(p);
        f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
    }
    __device__ static void store(float* p, const float (&f)[4]) { *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]); }
    __device__ static void store(__nv_bfloat16* p, const float (&f)[4]) {
        __nv_bfloat162 a = __floats2bfloat162_rn(f[0], f[1]), b = __floats2bfloat162_rn(f[2], f[3]);
        *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&b));
    }
};
template <> struct StreamVec<1> {
    __device__ static void load(const float* p, float (&f)[1]) { f[0] = p[0]; }
    __device__ static void store(float* p, const float (&f)[1]) { p[0] = f[0]; }
    __device__ static void store(__nv_bfloat16* p, const float (&f)[1]) { p[0] = __float2bfloat16_rn(f[0]); }
};

// VEC columns per access (4 when the width and the pointers allow); a thread keeps the u of kStepKeep accesses in
// registers (widths up to kStepKeep * VEC * 256) and forms u again from the new streams beyond that.
constexpr int kStepKeep = 4;

template <typename TO, int VEC>
__global__ void __launch_bounds__(kStreamThreads)
streams_step_kernel(float* __restrict__ x, const float* __restrict__ mix, const float* __restrict__ write,
                    float* __restrict__ y, const float* __restrict__ read, const float* __restrict__ w,
                    TO* __restrict__ out, int n_streams, int width, float eps) {
    __shared__ float scratch[33];
    __shared__ float m_s[kMaxStreams * kMaxStreams], w_s[kMaxStreams], r_s[kMaxStreams];
    for (int i = threadIdx.x; i < n_streams * n_streams; i += kStreamThreads) m_s[i] = mix[i];
    if (threadIdx.x < n_streams) {
        w_s[threadIdx.x] = write[threadIdx.x];
        r_s[threadIdx.x] = read != nullptr ? read[threadIdx.x] : 0.f;
    }
    __syncthreads();
    const size_t t = blockIdx.x;
    float* xr = x + t * n_streams * width;
    float* yr = y + t * width;
    const int units = width / VEC;
    float keep[kStepKeep][VEC];
    float ss = 0.f;
    auto column = [&](int c, float (&u)[VEC]) {
        float in[kMaxStreams][VEC], yv[VEC], zero[VEC];
#pragma unroll
        for (int a = 0; a < kMaxStreams; ++a)
            if (a < n_streams) StreamVec<VEC>::load(xr + (size_t)a * width + c, in[a]);
        StreamVec<VEC>::load(yr + c, yv);
#pragma unroll
        for (int e = 0; e < VEC; ++e) zero[e] = u[e] = 0.f;
        StreamVec<VEC>::store(yr + c, zero);
#pragma unroll
        for (int j = 0; j < kMaxStreams; ++j) {
            if (j >= n_streams) break;
            float acc[VEC];
#pragma unroll
            for (int e = 0; e < VEC; ++e) acc[e] = 0.f;
#pragma unroll
            for (int a = 0; a < kMaxStreams; ++a) {
                if (a >= n_streams) break;
                const float m = m_s[a * n_streams + j];
#pragma unroll
                for (int e = 0; e < VEC; ++e) acc[e] += m * in[a][e];
            }
#pragma unroll
            for (int e = 0; e < VEC; ++e) {
                acc[e] += w_s[j] * yv[e];
                u[e] += r_s[j] * acc[e];
            }
            StreamVec<VEC>::store(xr + (size_t)j * width + c, acc);
        }
    };
#pragma unroll
    for (int k = 0; k < kStepKeep; ++k) {
        const int unit = k * kStreamThreads + threadIdx.x;
#pragma unroll
        for (int e = 0; e < VEC; ++e) keep[k][e] = 0.f;
        if (unit < units) column(unit * VEC, keep[k]);
#pragma unroll
        for (int e = 0; e < VEC; ++e) ss += keep[k][e] * keep[k][e];
    }
    for (int unit = kStepKeep * kStreamThreads + threadIdx.x; unit < units; unit += kStreamThreads) {
        float u[VEC];
        column(unit * VEC, u);
#pragma unroll
        for (int e = 0; e < VEC; ++e) ss += u[e] * u[e];
    }
    if (read == nullptr) return;
    ss = block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)width + eps);
    TO* o = out + t * width;
#pragma unroll
    for (int k = 0; k < kStepKeep; ++k) {
        const int unit = k * kStreamThreads + threadIdx.x;
        if (unit < units) {
            float wv[VEC], res[VEC];
            StreamVec<VEC>::load(w + unit * VEC, wv);
#pragma unroll
            for (int e = 0; e < VEC; ++e) res[e] = wv[e] * (scale * keep[k][e]);
            StreamVec<VEC>::store(o + unit * VEC, res);
        }
    }
    for (int unit = kStepKeep * kStreamThreads + threadIdx.x; unit < units; unit += kStreamThreads) {
        float wv[VEC], res[VEC];   // beyond the kept columns u is formed again from the new streams (this thread wrote them)
        StreamVec<VEC>::load(w + unit * VEC, wv);
#pragma unroll
        for (int e = 0; e < VEC; ++e) res[e] = 0.f;
        for (int j = 0; j < n_streams; ++j) {
            float xv[VEC];
            StreamVec<VEC>::load(xr + (size_t)j * width + unit * VEC, xv);
#pragma unroll
            for (int e = 0; e < VEC; ++e) res[e] += r_s[j] * xv[e];
        }
#pragma unroll
        for (int e = 0; e < VEC; ++e) res[e] = wv[e] * (scale * res[e]);
        StreamVec<VEC>::store(o + unit * VEC, res);
    }
}

}  // namespace b200

extern "C" int b200_streams_step(float* x, const float* mix, const float* write, float* y, const float* read,
                                 const float* w, void* out, int out_dtype, int n_tokens, int n_streams, int width,
                                 float eps, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (n_streams < 1 || n_streams > b200::kMaxStreams || width < 1) return b200::kErrUnsupportedSize;
    if (read != nullptr && (w == nullptr || out == nullptr)) return b200::kErrBadArgument;
    const bool vec = width % 4 == 0 && (((uintptr_t)x | (uintptr_t)y | (uintptr_t)w | (uintptr_t)out) & 15) == 0;
    B200_DISPATCH_DTYPE(out_dtype, TO,
        if (vec) b200::streams_step_kernel<TO, 4><<<n_tokens, b200::kStreamThreads, 0, stream>>>(x, mix, write, y, read, w, (TO*)out, n_streams, width, eps);
        else b200::streams_step_kernel<TO, 1><<<n_tokens, b200::kStreamThreads, 0, stream>>>(x, mix, write, y, read, w, (TO*)out, n_streams, width, eps));
    return b200::launch_status();
}

extern "C" int b200_streams_combine(const float* x, float* out, const float* mix, const float* write, const float* y,
                                    int n_tokens, int s_in, int s_out, int width, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (s_in < 1 || s_out < 1 || s_in > b200::kMaxStreams || s_out > b200::kMaxStreams || width < 1) return b200::kErrUnsupportedSize;
    if (x == out && s_in != s_out) return b200::kErrBadArgument;
    const bool vec = width % 4 == 0 && (((uintptr_t)x | (uintptr_t)out | (uintptr_t)y) & 15) == 0;
    const size_t units = (size_t)n_tokens * width / (vec ? 4 : 1);
    const int grid = (int)((units + b200::kStreamThreads - 1) / b200::kStreamThreads < 148 * 16
                               ? (units + b200::kStreamThreads - 1) / b200::kStreamThreads : 148 * 16);
    if (vec) b200::streams_combine_kernel<4><<<grid, b200::kStreamThreads, 0, stream>>>(x, out, mix, write, y, s_in, s_out, width, units);
    else b200::streams_combine_kernel<1><<<grid, b200::kStreamThreads, 0, stream>>>(x, out, mix, write, y, s_in, s_out, width, units);
    return b200::launch_status();
}

extern "C" int b200_streams_read_norm(const float* x, const float* read, const float* w, void* out, int out_dtype,
                                      const int* rows, int n_rows, int n_streams, int width, float eps,
                                      cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (n_streams < 1 || n_streams > b200::kMaxStreams || width < 1) return b200::kErrUnsupportedSize;
    B200_DISPATCH_DTYPE(out_dtype, TO,
        b200::streams_read_norm_kernel<TO><<<n_rows, b200::kStreamThreads, 0, stream>>>(x, read, w, (TO*)out, rows,
                                                                                       n_streams, width, eps));
    return b200::launch_status();
}
