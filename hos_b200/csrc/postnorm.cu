// Row kernels of a block whose norm comes AFTER the residual sum, and of mixers that norm and gate
// their heads' outputs.
//
// scale_add_norm: x <- RMSNorm(alpha * x + y; w, eps), x the 32-bit residual stream, y a branch's output
//   (rows in any type, or 32-bit partial sums [parts][N][D] of a product that split K, added here in a
//   fixed order).  The same launch also writes what reads the new x next: h = x in the products' type
//   (the next branch reads x itself), or h = RMSNorm(x; w_next, eps_next) (the model's last norm).
// cast_rows: h = x in the products' type (the first layer's input).
// group_norm_gate: out[n][g][:] = o[n][g][:] / sqrt(mean_g(o^2) + eps) * w * act(gate[n][g][:]), the
//   groups being heads (a weight shared by all heads) or the whole row (one group, a weight per column);
//   act is the logistic function or x times it.  Statistics, weight and gate are 32-bit.
#include "common.cuh"

namespace hos {

template <typename TY, typename TH>
__global__ void __launch_bounds__(256)
scale_add_norm_kernel(const TY* __restrict__ y, int n_parts, long long part_stride, float alpha, float* __restrict__ x,
                      const float* __restrict__ w, float eps, TH* __restrict__ h, const float* __restrict__ w_next,
                      float eps_next, int D) {
    pdl_enter();
    extern __shared__ float row[];
    __shared__ float scratch[32];
    const size_t base = (size_t)blockIdx.x * D;
    float ss = 0.f;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float b = to_float(y[base + d]);
        for (int p = 1; p < n_parts; ++p) b += to_float(y[(size_t)p * part_stride + base + d]);
        const float s = fmaf(alpha, x[base + d], b);
        row[d] = s;
        ss = fmaf(s, s, ss);
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.f / sqrtf(ss / (float)D + eps);
    float ss2 = 0.f;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        const float v = row[d] * inv * w[d];
        x[base + d] = v;
        row[d] = v;
        ss2 = fmaf(v, v, ss2);
    }
    if (h == nullptr) return;
    if (w_next == nullptr) {
        for (int d = threadIdx.x; d < D; d += blockDim.x) h[base + d] = from_float<TH>(row[d]);
        return;
    }
    ss2 = block_sum(ss2, scratch);
    const float inv2 = 1.f / sqrtf(ss2 / (float)D + eps_next);
    for (int d = threadIdx.x; d < D; d += blockDim.x) h[base + d] = from_float<TH>(row[d] * inv2 * w_next[d]);
}

// The same with the row in registers: widths that are multiples of 4, up to 256 threads x NV x 4 numbers; 16-byte
// loads and stores of the 32-bit rows, 8-byte ones of bfloat16 rows.
__device__ __forceinline__ float4 load4(const float* p) { return *(const float4*)p; }
__device__ __forceinline__ float4 load4(const bf16* p) {
    const uint2 u = *(const uint2*)p;
    return make_float4(__uint_as_float(u.x << 16), __uint_as_float(u.x & 0xffff0000u), __uint_as_float(u.y << 16),
                       __uint_as_float(u.y & 0xffff0000u));
}
__device__ __forceinline__ void store4(float* p, float4 v) { *(float4*)p = v; }
__device__ __forceinline__ void store4(bf16* p, float4 v) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 u;
    u.x = *reinterpret_cast<uint32_t*>(&a);
    u.y = *reinterpret_cast<uint32_t*>(&b);
    *(uint2*)p = u;
}

template <typename TY, typename TH, int NV>
__global__ void __launch_bounds__(256)
scale_add_norm_vec_kernel(const TY* __restrict__ y, int n_parts, long long part_stride, float alpha, float* __restrict__ x,
                          const float* __restrict__ w, float eps, TH* __restrict__ h, const float* __restrict__ w_next,
                          float eps_next, int D) {
    pdl_enter();
    __shared__ float scratch[32];
    const size_t base = (size_t)blockIdx.x * D;
    float4 v[NV];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int d = (threadIdx.x + i * 256) * 4;
        v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (d < D) {
            float4 b = load4(y + base + d);
            for (int p = 1; p < n_parts; ++p) {
                const float4 c = load4(y + (size_t)p * part_stride + base + d);
                b.x += c.x; b.y += c.y; b.z += c.z; b.w += c.w;
            }
            const float4 xv = load4(x + base + d);
            v[i] = make_float4(fmaf(alpha, xv.x, b.x), fmaf(alpha, xv.y, b.y), fmaf(alpha, xv.z, b.z), fmaf(alpha, xv.w, b.w));
            ss += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
        }
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.f / sqrtf(ss / (float)D + eps);
    float ss2 = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int d = (threadIdx.x + i * 256) * 4;
        if (d < D) {
            const float4 wv = load4(w + d);
            v[i] = make_float4(v[i].x * inv * wv.x, v[i].y * inv * wv.y, v[i].z * inv * wv.z, v[i].w * inv * wv.w);
            store4(x + base + d, v[i]);
            ss2 += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
        }
    }
    if (h == nullptr) return;
    float inv2 = 1.f;
    if (w_next != nullptr) {
        ss2 = block_sum(ss2, scratch);
        inv2 = 1.f / sqrtf(ss2 / (float)D + eps_next);
    }
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int d = (threadIdx.x + i * 256) * 4;
        if (d < D) {
            float4 o = v[i];
            if (w_next != nullptr) {
                const float4 wv = load4(w_next + d);
                o = make_float4(o.x * inv2 * wv.x, o.y * inv2 * wv.y, o.z * inv2 * wv.z, o.w * inv2 * wv.w);
            }
            store4(h + base + d, o);
        }
    }
}

template <typename TH>
__global__ void cast_rows_kernel(const float* __restrict__ x, TH* __restrict__ h, long long n) {
    pdl_enter();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) h[i] = from_float<TH>(x[i]);
}

template <typename TH>
__global__ void __launch_bounds__(128)
group_norm_gate_kernel(const float* __restrict__ o, const float* __restrict__ w, int w_per_group,
                       const float* __restrict__ gate, long long gate_stride, int act, const int* __restrict__ token_seq,
                       TH* __restrict__ out, float eps, int G, int gs) {
    pdl_enter();
    __shared__ float scratch[32];
    const int n = blockIdx.x, g = blockIdx.y;
    const size_t base = ((size_t)n * G + g) * gs;
    if (token_seq != nullptr && token_seq[n] < 0) {        // padding: a defined row, nothing read
        for (int d = threadIdx.x; d < gs; d += blockDim.x) out[base + d] = from_float<TH>(0.f);
        return;
    }
    float ss = 0.f;
    for (int d = threadIdx.x; d < gs; d += blockDim.x) {
        const float v = o[base + d];
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.f / sqrtf(ss / (float)gs + eps);
    const float* wg = w + (w_per_group ? 0 : (size_t)g * gs);
    const float* gt = gate + (size_t)n * gate_stride + (size_t)g * gs;
    for (int d = threadIdx.x; d < gs; d += blockDim.x) {
        const float z = gt[d];
        const float s = 1.f / (1.f + expf(-z));
        out[base + d] = from_float<TH>(o[base + d] * inv * wg[d] * (act == 1 ? z * s : s));
    }
}

// The same with a warp to a group (heads of up to 2,048 numbers, a multiple of 4): a block takes a row, its warps the
// row's groups in turn; 16-byte reads, the group read twice (the second time from L1).
template <typename TH>
__global__ void __launch_bounds__(256)
group_norm_gate_warp_kernel(const float* __restrict__ o, const float* __restrict__ w, int w_per_group,
                            const float* __restrict__ gate, long long gate_stride, int act, const int* __restrict__ token_seq,
                            TH* __restrict__ out, float eps, int G, int gs) {
    pdl_enter();
    const int n = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool pad = token_seq != nullptr && token_seq[n] < 0;
    for (int g = warp; g < G; g += 8) {
        const size_t base = ((size_t)n * G + g) * gs;
        if (pad) {
            for (int d = lane * 4; d < gs; d += 128) store4(out + base + d, make_float4(0.f, 0.f, 0.f, 0.f));
            continue;
        }
        float ss = 0.f;
        for (int d = lane * 4; d < gs; d += 128) {
            const float4 v = load4(o + base + d);
            ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
        ss = warp_sum(ss);
        const float inv = 1.f / sqrtf(ss / (float)gs + eps);
        const float* wg = w + (w_per_group ? 0 : (size_t)g * gs);
        const float* gt = gate + (size_t)n * gate_stride + (size_t)g * gs;
        for (int d = lane * 4; d < gs; d += 128) {
            const float4 v = load4(o + base + d), wv = load4(wg + d), z = load4(gt + d);
            float4 r;
            const float s0 = 1.f / (1.f + expf(-z.x)), s1 = 1.f / (1.f + expf(-z.y)), s2 = 1.f / (1.f + expf(-z.z)),
                        s3 = 1.f / (1.f + expf(-z.w));
            r.x = v.x * inv * wv.x * (act == 1 ? z.x * s0 : s0);
            r.y = v.y * inv * wv.y * (act == 1 ? z.y * s1 : s1);
            r.z = v.z * inv * wv.z * (act == 1 ? z.z * s2 : s2);
            r.w = v.w * inv * wv.w * (act == 1 ? z.w * s3 : s3);
            store4(out + base + d, r);
        }
    }
}

}  // namespace hos

using namespace hos;

extern "C" const char* hos_last_error() { return error_buffer(); }

// y: [N][D] of y_dtype, or n_parts > 1 planes of float32 partial sums.  h (of h_dtype) may be null; with w_next
// null it is x itself in that type, else the next norm of x.
extern "C" int hos_scale_add_norm(const void* y, int y_dtype, int n_parts, float alpha, float* x, const float* w, float eps,
                                  void* h, int h_dtype, const float* w_next, float eps_next, int N, int D,
                                  cudaStream_t stream) {
    if (N <= 0) return 0;
    if (n_parts > 1 && y_dtype != kF32) HOS_REFUSE("scale_add_norm: partial sums must be float32");
    const size_t smem = (size_t)D * sizeof(float);
    if (smem > 200 * 1024) HOS_REFUSE("scale_add_norm: width %d does not fit a block's shared memory", D);
    const long long plane = (long long)N * D;
    const bool vec = D % 4 == 0 && D <= 256 * 4 * 8 && (uintptr_t)y % 16 == 0 && (uintptr_t)x % 16 == 0 &&
                     (h == nullptr || (uintptr_t)h % 16 == 0);
#define HOS_SAN_V(TY, TH, NV)                                                                                        \
    launch_pdl(scale_add_norm_vec_kernel<TY, TH, NV>, dim3(N), dim3(256), 0, stream, (const TY*)y, n_parts, plane, alpha, x, \
               w, eps, (TH*)h, w_next, eps_next, D)
#define HOS_SAN(TY, TH)                                                                                              \
    do {                                                                                                             \
        if (vec) {                                                                                                   \
            if (D <= 1024) HOS_SAN_V(TY, TH, 1);                                                                     \
            else if (D <= 2048) HOS_SAN_V(TY, TH, 2);                                                                \
            else if (D <= 4096) HOS_SAN_V(TY, TH, 4);                                                                \
            else HOS_SAN_V(TY, TH, 8);                                                                               \
            break;                                                                                                   \
        }                                                                                                            \
        if (smem > 48 * 1024)                                                                                        \
            cudaFuncSetAttribute(scale_add_norm_kernel<TY, TH>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        launch_pdl(scale_add_norm_kernel<TY, TH>, dim3(N), dim3(256), smem, stream, (const TY*)y, n_parts, plane, alpha, x, \
                   w, eps, (TH*)h, w_next, eps_next, D);                                                             \
    } while (0)
    const bool hb = h != nullptr && h_dtype == kBF16;
    if (y_dtype == kBF16 && hb) HOS_SAN(bf16, bf16);
    else if (y_dtype == kBF16) HOS_SAN(bf16, float);
    else if (hb) HOS_SAN(float, bf16);
    else HOS_SAN(float, float);
#undef HOS_SAN
#undef HOS_SAN_V
    return check_launch("scale_add_norm");
}

extern "C" int hos_cast_rows(const float* x, void* h, int h_dtype, long long n, cudaStream_t stream) {
    if (n <= 0) return 0;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (h_dtype == kBF16) launch_pdl(cast_rows_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, x, (bf16*)h, n);
    else launch_pdl(cast_rows_kernel<float>, dim3(blocks), dim3(256), 0, stream, x, (float*)h, n);
    return check_launch("cast_rows");
}

// o: [N][G][gs] float32.  w: [gs] if w_per_group (one weight for every group) else [G][gs].  gate: row n's gate of
// group g, column d at gate[n * gate_stride + g * gs + d].  act: 0 logistic, 1 x times logistic.
extern "C" int hos_group_norm_gate(const float* o, const float* w, int w_per_group, const float* gate, long long gate_stride,
                                   int act, const int* token_seq, void* out, int out_dtype, float eps, int N, int G, int gs,
                                   cudaStream_t stream) {
    if (N <= 0) return 0;
    if (G <= 0 || gs <= 0 || G > 65535) HOS_REFUSE("group_norm_gate: %d groups of %d", G, gs);
    if (G >= 2 && gs <= 2048 && gs % 4 == 0 && gate_stride % 4 == 0 && (uintptr_t)o % 16 == 0 && (uintptr_t)gate % 16 == 0 &&
        (uintptr_t)w % 16 == 0 && (uintptr_t)out % 16 == 0) {
        if (out_dtype == kBF16)
            launch_pdl(group_norm_gate_warp_kernel<bf16>, dim3(N), dim3(256), 0, stream, o, w, w_per_group, gate, gate_stride,
                       act, token_seq, (bf16*)out, eps, G, gs);
        else
            launch_pdl(group_norm_gate_warp_kernel<float>, dim3(N), dim3(256), 0, stream, o, w, w_per_group, gate, gate_stride,
                       act, token_seq, (float*)out, eps, G, gs);
        return check_launch("group_norm_gate");
    }
    if (out_dtype == kBF16)
        launch_pdl(group_norm_gate_kernel<bf16>, dim3(N, G), dim3(128), 0, stream, o, w, w_per_group, gate, gate_stride, act,
                   token_seq, (bf16*)out, eps, G, gs);
    else
        launch_pdl(group_norm_gate_kernel<float>, dim3(N, G), dim3(128), 0, stream, o, w, w_per_group, gate, gate_stride, act,
                   token_seq, (float*)out, eps, G, gs);
    return check_launch("group_norm_gate");
}
