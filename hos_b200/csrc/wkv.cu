// A linear-recurrence mixer with a matrix state per head (time mixing in the manner of RWKV).
//
// For every token t of a sequence, per head (size d), with r, k, v the projections, w the decay
// in (0, 1) per key channel and u a learned bonus for the current token:
//     o_t = (S_{t-1} + diag(u) k_t v_t^T)^T r_t
//     S_t = diag(w_t) S_{t-1} + k_t v_t^T                        S: [d keys][d values], 32-bit
// then o_t / sqrt(mean(o_t^2) + eps) * norm_weight * silu(g_t), which the output projection reads.
// The decay is w_t = exp(-exp(x_t + w0)) with x_t the low-rank projection that the host runs
// between the two kernels here; all of it 32-bit.
//
// token_shift: the five inputs of the projections, mix_s[t] = h_t + (h_{t-1} - h_t) * mu_s, with
// h_{t-1} = 0 for a sequence's first token and the kept row (state, one per slot) for the first row
// of a step that continues a sequence.
// wkv_scan: one block per (sequence, head), thread j owns column j of S (in shared memory), tokens
// in order; starts from the slot's state (from zero for a sequence whose first row is position 0),
// leaves the new state there, and keeps the step's last h row for the next step's token shift.
#include "common.cuh"

namespace hos {

template <typename T>
__global__ void token_shift_kernel(const T* __restrict__ h, const float* __restrict__ kept, const float* __restrict__ mu,
                                   int n_mix, const int* __restrict__ token_pos, const int* __restrict__ token_seq,
                                   const int* __restrict__ cu_seqlens, const int* __restrict__ seq_slot,
                                   T* __restrict__ out, long long plane, int D) {
    pdl_enter();
    const int n = blockIdx.x;
    const int seq = token_seq[n];
    if (seq < 0) {
        for (int d = threadIdx.x; d < D; d += blockDim.x)
            for (int s = 0; s < n_mix; ++s) out[s * plane + (size_t)n * D + d] = from_float<T>(0.f);
        return;
    }
    const bool first_row = n == cu_seqlens[seq];
    const bool from_zero = token_pos[n] == 0;
    const float* keep = kept + (size_t)seq_slot[seq] * D;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        const float cur = to_float(h[(size_t)n * D + d]);
        const float prev = from_zero ? 0.f : (first_row ? keep[d] : to_float(h[(size_t)(n - 1) * D + d]));
        const float diff = prev - cur;
        for (int s = 0; s < n_mix; ++s) out[s * plane + (size_t)n * D + d] = from_float<T>(fmaf(diff, mu[s * D + d], cur));
    }
}

template <typename T>
__global__ void tanh_rows_kernel(const float* __restrict__ x, T* __restrict__ out, long long n) {
    pdl_enter();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = from_float<T>(tanhf(x[i]));
}

template <typename T>
__global__ void wkv_scan_kernel(const float* __restrict__ r, const float* __restrict__ k, const float* __restrict__ v,
                                const float* __restrict__ wx, const float* __restrict__ g, const float* __restrict__ w0,
                                const float* __restrict__ u, const float* __restrict__ norm_w, float eps,
                                float* __restrict__ state, float* __restrict__ kept, const T* __restrict__ h, int width,
                                const int* __restrict__ token_pos, const int* __restrict__ token_seq,
                                const int* __restrict__ cu_seqlens, const int* __restrict__ seq_slot,
                                T* __restrict__ out, int H, int d) {
    pdl_enter();
    extern __shared__ float sm[];
    float* S = sm;                    // [d][d]
    float* rs = S + d * d;            // [d] each
    float* ks = rs + d;
    float* ws = ks + d;
    float* us = ws + d;
    __shared__ float scratch[32];
    const int seq = blockIdx.x, head = blockIdx.y, j = threadIdx.x;
    const int lo = cu_seqlens[seq];
    int hi = cu_seqlens[seq + 1];
    if (hi <= lo || token_seq[lo] < 0) return;
    const int slot = seq_slot[seq];
    const int C = H * d;
    float* st = state + ((size_t)slot * H + head) * d * d;
    const bool fresh = token_pos[lo] == 0;
    const bool mine = j < d;
    if (mine) {
        for (int i = 0; i < d; ++i) S[i * d + j] = fresh ? 0.f : st[i * d + j];
        us[j] = u[head * d + j];
    }
    const float nw = mine ? norm_w[head * d + j] : 0.f;
    const float w0j = mine ? w0[head * d + j] : 0.f;
    for (int t = lo; t < hi; ++t) {
        const size_t at = (size_t)t * C + head * d + j;
        float vj = 0.f, gj = 0.f;
        if (mine) {
            rs[j] = r[at];
            ks[j] = k[at];
            ws[j] = expf(-expf(wx[at] + w0j));
            vj = v[at];
            gj = g[at];
        }
        __syncthreads();
        float acc = 0.f;
        if (mine) {
            for (int i = 0; i < d; ++i) {
                const float s = S[i * d + j];
                const float kv = ks[i] * vj;
                acc = fmaf(rs[i], fmaf(us[i], kv, s), acc);
                S[i * d + j] = fmaf(ws[i], s, kv);
            }
        }
        const float ss = block_sum(acc * acc, scratch);      // its barriers also end this token's reads of rs, ks, ws
        if (mine) {
            const float gate = gj / (1.f + expf(-gj));
            out[at] = from_float<T>(acc * rsqrtf(ss / (float)d + eps) * nw * gate);
        }
    }
    if (mine)
        for (int i = 0; i < d; ++i) st[i * d + j] = S[i * d + j];
    if (head == 0)                    // the row that the next step's first token is shifted against
        for (int c = j; c < width; c += blockDim.x) kept[(size_t)slot * width + c] = to_float(h[(size_t)(hi - 1) * width + c]);
}

// The same walk with the state in registers, for the head sizes that are compiled in (D).  A column of S is cut
// into kParts runs of rows, one thread each (thread = (part, column)), so that a head keeps kParts * D threads
// busy; the parts' sums are added when the head norm is taken.  The tokens come in chunks whose r, k, decay, v
// and gate rows are brought to shared memory together, so that a chunk costs three barriers instead of three per
// token; the head norm's sums are taken per chunk, a warp per token.
template <int D> struct ScanShape {
    static constexpr int kParts = D <= 16 ? 4 : (D <= 32 ? 8 : (D <= 64 ? 4 : 2));
    static constexpr int kRows = D / kParts;               // rows of S per thread (a multiple of 4)
    static constexpr int kThreads = (kParts * D + 31) / 32 * 32;
    static constexpr int kChunk = D <= 64 ? 16 : 8;
};

template <typename T, int D>
__global__ void __launch_bounds__(ScanShape<D>::kThreads)
wkv_scan_reg_kernel(const float* __restrict__ r, const float* __restrict__ k, const float* __restrict__ v,
                    const float* __restrict__ wx, const float* __restrict__ g, const float* __restrict__ w0,
                    const float* __restrict__ u, const float* __restrict__ norm_w, float eps,
                    float* __restrict__ state, float* __restrict__ kept, const T* __restrict__ h, int width,
                    const int* __restrict__ token_pos, const int* __restrict__ token_seq,
                    const int* __restrict__ cu_seqlens, const int* __restrict__ seq_slot, T* __restrict__ out, int H) {
    pdl_enter();
    constexpr int kParts = ScanShape<D>::kParts, kRows = ScanShape<D>::kRows, kThreads = ScanShape<D>::kThreads,
                  kChunk = ScanShape<D>::kChunk;
    static_assert(kRows % 4 == 0 && kRows * kParts == D, "a thread's rows come four at a time");
    __shared__ __align__(16) float rs[kChunk][D], ks[kChunk][D], ws[kChunk][D], vs[kChunk][D], gs[kChunk][D],
        os[kParts][kChunk][D], us[D], scale[kChunk];
    const int seq = blockIdx.x, head = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int j = tid % D, part = tid / D, i0 = part * kRows;
    const int lo = cu_seqlens[seq], hi = cu_seqlens[seq + 1];
    if (hi <= lo || token_seq[lo] < 0) return;
    const int slot = seq_slot[seq];
    const int C = H * D;
    float* st = state + ((size_t)slot * H + head) * D * D;
    const bool fresh = token_pos[lo] == 0;
    const bool mine = part < kParts;
    float S[kRows];
#pragma unroll
    for (int i = 0; i < kRows; ++i) S[i] = (mine && !fresh) ? st[(i0 + i) * D + j] : 0.f;
    if (tid < D) us[tid] = u[head * D + tid];
    for (int t0 = lo; t0 < hi; t0 += kChunk) {
        const int nt = min(kChunk, hi - t0);
        for (int x = tid; x < nt * D; x += kThreads) {
            const int t = x / D, c = x - t * D;
            const size_t at = (size_t)(t0 + t) * C + head * D + c;
            rs[t][c] = r[at];
            ks[t][c] = k[at];
            ws[t][c] = expf(-expf(wx[at] + w0[head * D + c]));
            vs[t][c] = v[at];
            gs[t][c] = g[at];
        }
        __syncthreads();
        if (mine) {
            for (int t = 0; t < nt; ++t) {
                float acc[4] = {0.f, 0.f, 0.f, 0.f};          // four chains: the sum does not wait for itself
                const float vt = vs[t][j];
#pragma unroll
                for (int i = 0; i < kRows; i += 4) {
                    const float4 k4 = *reinterpret_cast<const float4*>(&ks[t][i0 + i]);
                    const float4 r4 = *reinterpret_cast<const float4*>(&rs[t][i0 + i]);
                    const float4 w4 = *reinterpret_cast<const float4*>(&ws[t][i0 + i]);
                    const float4 u4 = *reinterpret_cast<const float4*>(&us[i0 + i]);
                    const float kv0 = k4.x * vt, kv1 = k4.y * vt, kv2 = k4.z * vt, kv3 = k4.w * vt;
                    acc[0] = fmaf(r4.x, fmaf(u4.x, kv0, S[i]), acc[0]);
                    acc[1] = fmaf(r4.y, fmaf(u4.y, kv1, S[i + 1]), acc[1]);
                    acc[2] = fmaf(r4.z, fmaf(u4.z, kv2, S[i + 2]), acc[2]);
                    acc[3] = fmaf(r4.w, fmaf(u4.w, kv3, S[i + 3]), acc[3]);
                    S[i] = fmaf(w4.x, S[i], kv0);
                    S[i + 1] = fmaf(w4.y, S[i + 1], kv1);
                    S[i + 2] = fmaf(w4.z, S[i + 2], kv2);
                    S[i + 3] = fmaf(w4.w, S[i + 3], kv3);
                }
                os[part][t][j] = (acc[0] + acc[1]) + (acc[2] + acc[3]);
            }
        }
        __syncthreads();
        for (int t = warp; t < nt; t += kThreads / 32) {
            float ss = 0.f;
            for (int i = lane; i < D; i += 32) {
                float o = os[0][t][i];
#pragma unroll
                for (int p = 1; p < kParts; ++p) o += os[p][t][i];
                os[0][t][i] = o;
                ss = fmaf(o, o, ss);
            }
            ss = warp_sum(ss);
            if (lane == 0) scale[t] = rsqrtf(ss / (float)D + eps);
        }
        __syncthreads();
        for (int x = tid; x < nt * D; x += kThreads) {
            const int t = x / D, c = x - t * D;
            const float gt = gs[t][c];
            out[(size_t)(t0 + t) * C + head * D + c] =
                from_float<T>(os[0][t][c] * scale[t] * norm_w[head * D + c] * (gt / (1.f + expf(-gt))));
        }
        __syncthreads();          // the next chunk's rows overwrite what this one has just read
    }
    if (mine) {
#pragma unroll
        for (int i = 0; i < kRows; ++i) st[(i0 + i) * D + j] = S[i];
    }
    if (head == 0)
        for (int c = tid; c < width; c += kThreads) kept[(size_t)slot * width + c] = to_float(h[(size_t)(hi - 1) * width + c]);
}

template <typename T>
static bool launch_scan_reg(int d, dim3 grid, cudaStream_t stream, const float* r, const float* k, const float* v,
                            const float* wx, const float* g, const float* w0, const float* u, const float* norm_w,
                            float eps, float* state, float* kept, const void* h, int width, const int* token_pos,
                            const int* token_seq, const int* cu_seqlens, const int* seq_slot, void* out, int H) {
#define HOS_SCAN(DD)                                                                                                  \
    if (d == DD) {                                                                                                    \
        launch_pdl(wkv_scan_reg_kernel<T, DD>, grid, dim3(ScanShape<DD>::kThreads), 0, stream, r, k, v, wx, g, w0, u,     \
                   norm_w, eps, state, kept, (const T*)h, width, token_pos, token_seq, cu_seqlens, seq_slot, (T*)out, H); \
        return true;                                                                                                  \
    }
    HOS_SCAN(16) HOS_SCAN(32) HOS_SCAN(48) HOS_SCAN(64) HOS_SCAN(96) HOS_SCAN(128)
#undef HOS_SCAN
    return false;
}

}  // namespace hos

using namespace hos;

// out: n_mix planes of [N][D] of the activations' type, `plane` elements apart; mu: [n_mix][D]; kept: [slots][D] 32-bit.
extern "C" int hos_token_shift(const void* h, int dtype, const float* kept, const float* mu, int n_mix,
                               const int* token_pos, const int* token_seq, const int* cu_seqlens,
                               const int* seq_slot, void* out, long long plane, int N, int D, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (plane < (long long)N * D) HOS_REFUSE("token_shift: the planes overlap");
    if (dtype == kBF16)
        launch_pdl(token_shift_kernel<bf16>, dim3(N), dim3(128), 0, stream, (const bf16*)h, kept, mu, n_mix, token_pos,
                   token_seq, cu_seqlens, seq_slot, (bf16*)out, plane, D);
    else if (dtype == kF32)
        launch_pdl(token_shift_kernel<float>, dim3(N), dim3(128), 0, stream, (const float*)h, kept, mu, n_mix, token_pos,
                   token_seq, cu_seqlens, seq_slot, (float*)out, plane, D);
    else
        HOS_REFUSE("token_shift: unknown dtype %d", dtype);
    return check_launch("token_shift");
}

extern "C" int hos_tanh_rows(const float* x, void* out, int out_dtype, long long n, cudaStream_t stream) {
    if (n <= 0) return 0;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (out_dtype == kBF16) launch_pdl(tanh_rows_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, x, (bf16*)out, n);
    else if (out_dtype == kF32) launch_pdl(tanh_rows_kernel<float>, dim3(blocks), dim3(256), 0, stream, x, (float*)out, n);
    else HOS_REFUSE("tanh_rows: unknown dtype %d", out_dtype);
    return check_launch("tanh_rows");
}

// r, k, v, wx, g: [N][H*d] 32-bit; state: [slots][H][d][d]; kept: [slots][width]; h: [N][width]; out: [N][H*d].
extern "C" int hos_wkv_scan(const float* r, const float* k, const float* v, const float* wx, const float* g,
                            const float* w0, const float* u, const float* norm_w, float eps, float* state,
                            float* kept, const void* h, int dtype, int width, const int* token_pos,
                            const int* token_seq, const int* cu_seqlens, const int* seq_slot, void* out,
                            int n_seqs, int H, int d, cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    const size_t smem = (size_t)(d * d + 4 * d) * sizeof(float);
    if (d > 1024 || smem > 200 * 1024) HOS_REFUSE("wkv_scan: a head of %d does not fit a block's shared memory", d);
    const int threads = (d + 31) / 32 * 32;
    if (dtype == kBF16 && launch_scan_reg<bf16>(d, dim3(n_seqs, H), stream, r, k, v, wx, g, w0, u, norm_w, eps, state, kept, h,
                                                width, token_pos, token_seq, cu_seqlens, seq_slot, out, H))
        return check_launch("wkv_scan");
    if (dtype == kF32 && launch_scan_reg<float>(d, dim3(n_seqs, H), stream, r, k, v, wx, g, w0, u, norm_w, eps, state, kept, h,
                                                width, token_pos, token_seq, cu_seqlens, seq_slot, out, H))
        return check_launch("wkv_scan");
    if (dtype == kBF16) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(wkv_scan_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        launch_pdl(wkv_scan_kernel<bf16>, dim3(n_seqs, H), dim3(threads), smem, stream, r, k, v, wx, g, w0, u, norm_w, eps,
                   state, kept, (const bf16*)h, width, token_pos, token_seq, cu_seqlens, seq_slot, (bf16*)out, H, d);
    } else if (dtype == kF32) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(wkv_scan_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        launch_pdl(wkv_scan_kernel<float>, dim3(n_seqs, H), dim3(threads), smem, stream, r, k, v, wx, g, w0, u, norm_w, eps,
                   state, kept, (const float*)h, width, token_pos, token_seq, cu_seqlens, seq_slot, (float*)out, H, d);
    } else {
        HOS_REFUSE("wkv_scan: unknown dtype %d", dtype);
    }
    return check_launch("wkv_scan");
}
