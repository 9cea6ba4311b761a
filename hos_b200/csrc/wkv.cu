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
