// Token embedding with a hashed token-pair table, and the parallel block's row kernel.
//
// embed_pair: x[n] = table[token] + pair_table[row], where row is
//   (previous token * mul_prev + token * mul_cur) mod buckets
// and, for a sequence's first token, row `buckets` (the table's last row).  The previous token
// of a step's first row of a sequence that is under way comes from the sequence's state (one
// int per slot), which keep_last_token moves on after the step's rows have been read.
//
// scaled_add_norms: x += mult * (a + f), then up to two RMS norms of the new x with weights of
// their own (h1 = x / sqrt(mean(x^2) + eps1) * w1, h2 likewise): what a block needs whose mixer
// and feed-forward both read a norm of the same x.  Sums, statistics and x are 32-bit.
#include "common.cuh"

namespace hos {

__device__ __forceinline__ float load_any(const void* p, int dtype, size_t i) {
    return dtype == kBF16 ? to_float(((const bf16*)p)[i]) : ((const float*)p)[i];
}
__device__ __forceinline__ void store_any(void* p, int dtype, size_t i, float v) {
    if (dtype == kBF16) ((bf16*)p)[i] = from_float<bf16>(v);
    else ((float*)p)[i] = v;
}

template <typename TW>
__global__ void embed_pair_kernel(const int* __restrict__ tokens, const int* __restrict__ token_pos,
                                  const int* __restrict__ token_seq, const int* __restrict__ cu_seqlens,
                                  const int* __restrict__ seq_slot, const int* __restrict__ prev_token,
                                  const TW* __restrict__ table, const TW* __restrict__ pair_table, int buckets,
                                  long long mul_prev, long long mul_cur, float* __restrict__ out, int D) {
    pdl_enter();
    const int n = blockIdx.x;
    const int tok = tokens[n], seq = token_seq[n];
    float* o = out + (size_t)n * D;
    if (tok < 0 || seq < 0) {                 // padding: a zero row
        for (int d = threadIdx.x; d < D; d += blockDim.x) o[d] = 0.f;
        return;
    }
    int row = buckets;
    if (token_pos[n] > 0) {
        const int prev = n == cu_seqlens[seq] ? prev_token[seq_slot[seq]] : tokens[n - 1];
        long long r = ((long long)prev * mul_prev + (long long)tok * mul_cur) % (long long)buckets;
        if (r < 0) r += buckets;
        row = (int)r;
    }
    const TW* e = table + (size_t)tok * D;
    const TW* p = pair_table + (size_t)row * D;
    for (int d = threadIdx.x; d < D; d += blockDim.x) o[d] = to_float(e[d]) + to_float(p[d]);
}

// prev_token[slot of s] = the last token that sequence s brought (sequences without live rows are left alone)
__global__ void keep_last_token_kernel(const int* __restrict__ tokens, const int* __restrict__ token_seq,
                                       const int* __restrict__ cu_seqlens, const int* __restrict__ seq_slot,
                                       int* __restrict__ prev_token, int n_seqs) {
    pdl_enter();
    const int s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s >= n_seqs) return;
    const int lo = cu_seqlens[s], hi = cu_seqlens[s + 1];
    if (hi <= lo || token_seq[hi - 1] < 0 || tokens[hi - 1] < 0) return;
    prev_token[seq_slot[s]] = tokens[hi - 1];
}

__global__ void scaled_add_norms_kernel(const void* __restrict__ a, int a_dtype, const void* __restrict__ f,
                                        int f_dtype, float mult, float* __restrict__ x,
                                        const float* __restrict__ w1, float eps1, void* __restrict__ h1,
                                        const float* __restrict__ w2, float eps2, void* __restrict__ h2,
                                        int h_dtype, int D) {
    pdl_enter();
    extern __shared__ float row[];
    __shared__ float scratch[32];
    const size_t base = (size_t)blockIdx.x * D;
    float ss = 0.f;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float v = x[base + d];
        if (a != nullptr || f != nullptr) {
            float s = a != nullptr ? load_any(a, a_dtype, base + d) : 0.f;
            if (f != nullptr) s += load_any(f, f_dtype, base + d);
            v = fmaf(mult, s, v);
            x[base + d] = v;
        }
        row[d] = v;
        ss = fmaf(v, v, ss);
    }
    if (h1 == nullptr && h2 == nullptr) return;
    const float mean = block_sum(ss, scratch) / (float)D;
    const float r1 = rsqrtf(mean + eps1), r2 = rsqrtf(mean + eps2);
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        const float v = row[d];
        if (h1 != nullptr) store_any(h1, h_dtype, base + d, v * r1 * w1[d]);
        if (h2 != nullptr) store_any(h2, h_dtype, base + d, v * r2 * w2[d]);
    }
}

}  // namespace hos

using namespace hos;

extern "C" const char* hos_last_error() { return error_buffer(); }

extern "C" int hos_embed_pair(const int* tokens, const int* token_pos, const int* token_seq, const int* cu_seqlens,
                              const int* seq_slot, const int* prev_token, const void* table, const void* pair_table,
                              int table_dtype, int buckets, long long mul_prev, long long mul_cur, float* out,
                              int N, int D, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (buckets <= 0) HOS_REFUSE("embed_pair: the pair table needs at least one bucket");
    if (table_dtype == kBF16)
        launch_pdl(embed_pair_kernel<bf16>, dim3(N), dim3(128), 0, stream, tokens, token_pos, token_seq, cu_seqlens,
                   seq_slot, prev_token, (const bf16*)table, (const bf16*)pair_table, buckets, mul_prev, mul_cur, out, D);
    else if (table_dtype == kF32)
        launch_pdl(embed_pair_kernel<float>, dim3(N), dim3(128), 0, stream, tokens, token_pos, token_seq, cu_seqlens,
                   seq_slot, prev_token, (const float*)table, (const float*)pair_table, buckets, mul_prev, mul_cur, out, D);
    else
        HOS_REFUSE("embed_pair: unknown table dtype %d", table_dtype);
    return check_launch("embed_pair");
}

extern "C" int hos_keep_last_token(const int* tokens, const int* token_seq, const int* cu_seqlens,
                                   const int* seq_slot, int* prev_token, int n_seqs, cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    launch_pdl(keep_last_token_kernel, dim3((n_seqs + 127) / 128), dim3(128), 0, stream, tokens, token_seq,
               cu_seqlens, seq_slot, prev_token, n_seqs);
    return check_launch("keep_last_token");
}

// a, f: [N, D] of their dtypes or null; h1, h2: [N, D] of h_dtype or null.
extern "C" int hos_scaled_add_norms(const void* a, int a_dtype, const void* f, int f_dtype, float mult, float* x,
                                    const float* w1, float eps1, void* h1, const float* w2, float eps2, void* h2,
                                    int h_dtype, int N, int D, cudaStream_t stream) {
    if (N <= 0) return 0;
    const size_t smem = (size_t)D * sizeof(float);
    if (smem > 200 * 1024) HOS_REFUSE("scaled_add_norms: width %d does not fit a block's shared memory", D);
    if (smem > 48 * 1024)
        cudaFuncSetAttribute(scaled_add_norms_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_pdl(scaled_add_norms_kernel, dim3(N), dim3(256), smem, stream, a, a_dtype, f, f_dtype, mult, x, w1, eps1,
               h1, w2, eps2, h2, h_dtype, D);
    return check_launch("scaled_add_norms");
}
