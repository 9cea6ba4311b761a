// A 64 x 64 tile of a bfloat16 matrix product on the tensor cores (mma.sync m16n8k16, 32-bit accumulators),
// shared by the kernels whose rows are chosen on the device (the routed experts' products, the per-head
// products of the latent attention).  K runs in steps of 64 through a ring of kStages shared-memory stages
// filled by 16-byte asynchronous copies; a stage holds the 64 rows of A and NB weight tiles of 64 rows each, all
// as rows of 128 bytes whose 16-byte groups are XOR-permuted by the row, so that ldmatrix reads without bank
// conflicts.  8 warps as 4 (rows) x 2 (features).  A warp whose 16 rows are all padding issues no MMA.
// K and the operands' row strides must be multiples of 8 (16-byte rows).
#pragma once
#include "common.cuh"
#include "mma_utils.cuh"

namespace hos {

constexpr int kTile = 64;
constexpr int kStages = 3, kBK = 64;

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
    const int bytes = valid ? 16 : 0;            // 0: the 16 bytes are filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst)), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// element offset of (row, 16-byte group) in a tile of rows of 64 bf16
__device__ __forceinline__ int swz(int row, int group) { return row * kBK + ((group ^ (row & 7)) << 3); }

// NB: 1 (one weight tile) or 2 (two weight tiles, the second `second_tile_offset` elements further on: gate and up)
template <int NB>
struct TcTile {
    // stage layout: A [64][64], then NB weight tiles [64][64]
    static constexpr int kStageElems = (1 + NB) * kTile * kBK;
    static constexpr int kSmemBytes = kStages * kStageElems * 2;
};

template <int NB, typename RowPtr>
__device__ __forceinline__ void tc_mainloop(bf16* smem, RowPtr a_row, const bf16* __restrict__ W, int w_rows, int n0,
                                            size_t second_tile_offset, int K, bool busy, float (&acc)[NB][4][4]) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int warp_m = warp & 3, warp_n = warp >> 2;
    const int KT = (K + kBK - 1) / kBK;
    auto load = [&](int kt, int stage) {
        bf16* A = smem + stage * TcTile<NB>::kStageElems;
        const int k0 = kt * kBK;
        for (int x = tid; x < kTile * 8; x += 256) {
            const int r = x >> 3, g = x & 7, k = k0 + g * 8;
            const bf16* src = a_row(r);
            cp_async16(A + swz(r, g), src ? src + k : (const bf16*)W, src != nullptr && k < K);
        }
#pragma unroll
        for (int b = 0; b < NB; ++b) {
            bf16* B = A + (1 + b) * kTile * kBK;
            const bf16* Wb = W + b * second_tile_offset;
            for (int x = tid; x < kTile * 8; x += 256) {
                const int r = x >> 3, g = x & 7, k = k0 + g * 8, n = n0 + r;
                const bool ok = n < w_rows && k < K;
                cp_async16(B + swz(r, g), ok ? Wb + (size_t)n * K + k : W, ok);
            }
        }
    };
    for (int s = 0; s < kStages - 1; ++s) {
        if (s < KT) load(s, s);
        cp_async_commit();
    }
    for (int kt = 0; kt < KT; ++kt) {
        cp_async_wait<kStages - 2>();
        __syncthreads();
        if (kt + kStages - 1 < KT) load(kt + kStages - 1, (kt + kStages - 1) % kStages);
        cp_async_commit();
        if (!busy) continue;
        const bf16* A = smem + (kt % kStages) * TcTile<NB>::kStageElems;
#pragma unroll
        for (int ks = 0; ks < kBK / 16; ++ks) {
            uint32_t a[4];
            ldmatrix_x4(a, smem_u32(A + swz(warp_m * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, ks * 2 + (lane >> 4))));
#pragma unroll
            for (int b = 0; b < NB; ++b) {
                const bf16* B = A + (1 + b) * kTile * kBK;
#pragma unroll
                for (int np = 0; np < 2; ++np) {          // two pairs of 8-wide feature tiles
                    uint32_t w[4];
                    ldmatrix_x4(w, smem_u32(B + swz(warp_n * 32 + np * 16 + (lane & 7) + (lane >> 4) * 8,
                                                    ks * 2 + ((lane >> 3) & 1))));
                    mma_bf16(acc[b][np * 2], a, w[0], w[1]);
                    mma_bf16(acc[b][np * 2 + 1], a, w[2], w[3]);
                }
            }
        }
    }
    cp_async_wait<0>();
}


}  // namespace hos
