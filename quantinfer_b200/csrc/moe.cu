// Mixture of experts: routing, grouping of the tokens by expert, the experts' products as one grouped
// launch, and the weighted sum.
//
//   moe_route     per token: s = softmax(router logits) over all experts (32-bit); the `top` experts with the
//                 largest s + correction are chosen (ties: the lower index); their weights are their s divided
//                 by the sum of the chosen s (+ 1e-20) and multiplied by `scale`.
//   moe_group     the (token, choice) pairs sorted by expert: offsets per expert, the pairs' order, each pair's
//                 place in that order, and a list of row tiles (expert, first row, rows) of at most `tile` rows
//                 that no expert shares with another. One block; everything stays on the device, so a step
//                 never waits for the host to learn how many tokens an expert got.
//   moe_gemm      y[i] = W[expert of row i] . x[source of row i] over the sorted rows i, 32-bit products and
//                 sums with k ascending (the 32-bit path, and any type the tensor-core kernel does not take);
//                 a row's result does not depend on which other rows its expert got.
//   moe_combine   out[t] = sum_k weight[t, k] * y[place of (t, k)] (+ shared[t]), k ascending, 32-bit.
#include "common.cuh"

#include <math.h>

namespace {

constexpr int kMaxPerLane = 32;   // experts a lane holds: up to 1,024 experts

__global__ void __launch_bounds__(128)
moe_route_kernel(const float* __restrict__ logits, const float* __restrict__ correction, int* __restrict__ ids,
                 float* __restrict__ weights, int n, int E, int top, float scale) {
    qi::pdl_wait();
    const int t = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (t >= n) return;
    const float* z = logits + (size_t)t * E;
    float s[kMaxPerLane], c[kMaxPerLane];
    float m = -INFINITY;
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) {
        const int e = lane + 32 * i;
        s[i] = e < E ? z[e] : -INFINITY;
        m = fmaxf(m, s[i]);
    }
    m = qi::warp_max(m);
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) {
        const int e = lane + 32 * i;
        s[i] = e < E ? expf(s[i] - m) : 0.f;
        sum += s[i];
    }
    sum = qi::warp_sum(sum);
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) {
        const int e = lane + 32 * i;
        s[i] = s[i] / sum;
        c[i] = e < E ? s[i] + (correction ? correction[e] : 0.f) : -INFINITY;
    }
    float chosen_sum = 0.f;
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int best_e = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < kMaxPerLane; ++i) {
            const int e = lane + 32 * i;
            if (c[i] > best) { best = c[i]; best_e = e; }      // e ascends with i: the lower index wins a tie
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
            if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
        }
        if (best_e >= E) best_e = k % E;      // scores that are not numbers: any valid expert, so that what follows stays in range
        float sc = 0.f;
#pragma unroll
        for (int i = 0; i < kMaxPerLane; ++i)
            if (lane + 32 * i == best_e) { sc = s[i]; c[i] = -INFINITY; }
        sc = qi::warp_sum(sc);
        chosen_sum += sc;
        if ((k & 31) == lane) {      // lane k mod 32 writes choice k and scales it below
            ids[(size_t)t * top + k] = best_e;
            weights[(size_t)t * top + k] = sc;
        }
    }
    const float inv = scale / (chosen_sum + 1e-20f);
    for (int k = lane; k < top; k += 32) weights[(size_t)t * top + k] *= inv;
}

// One block. smem: counts[E], offsets[E + 1], tile_base[E + 1].
__global__ void __launch_bounds__(1024)
moe_group_kernel(const int* __restrict__ ids, int n_pairs, int E, int tile, int max_tiles, int* __restrict__ offsets,
                 int* __restrict__ order, int* __restrict__ place, int* __restrict__ tiles) {
    extern __shared__ int sm[];
    int* counts = sm;
    int* offs = sm + E;
    int* tbase = offs + E + 1;
    qi::pdl_wait();
    for (int e = threadIdx.x; e < E; e += blockDim.x) counts[e] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) {
        const int e = ids[i];
        if (e >= 0 && e < E) atomicAdd(&counts[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int a = 0, b = 0;
        for (int e = 0; e < E; ++e) {
            offs[e] = a; tbase[e] = b;
            a += counts[e];
            b += (counts[e] + tile - 1) / tile;
        }
        offs[E] = a; tbase[E] = b;
    }
    __syncthreads();
    for (int e = threadIdx.x; e <= E; e += blockDim.x) offsets[e] = offs[e];
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        const int cnt = counts[e];
        int k = tbase[e];
        for (int r0 = 0; r0 < cnt; r0 += tile, ++k) {
            if (k < max_tiles) { tiles[3 * k] = e; tiles[3 * k + 1] = offs[e] + r0; tiles[3 * k + 2] = min(tile, cnt - r0); }
        }
    }
    for (int k = tbase[E] + threadIdx.x; k < max_tiles; k += blockDim.x) { tiles[3 * k] = -1; tiles[3 * k + 1] = 0; tiles[3 * k + 2] = 0; }
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x) counts[e] = offs[e];     // cursors
    __syncthreads();
    for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) {
        const int e = ids[i];
        if (e < 0 || e >= E) continue;
        const int pos = atomicAdd(&counts[e], 1);
        order[pos] = i;
        place[i] = pos;
    }
}

constexpr int BM = 32, BN = 64, BK = 16, TM = 2, TN = 4;

// Rows are the sorted (token, choice) pairs; a tile's rows belong to one expert. Source row of sorted row i:
// order[i] / top when `gather` (the experts read the tokens' rows), else i (they read rows already in sorted order).
template <typename TX, typename TW, typename TY>
__global__ void __launch_bounds__(256)
moe_gemm_kernel(const TX* __restrict__ x, const TW* __restrict__ w, TY* __restrict__ y, const int* __restrict__ tiles,
                const int* __restrict__ order, int top, int gather, int N, int K, long long ldx, long long ldy, int n_src,
                int n_rows, int n_experts) {
    __shared__ float xs[BK][BM + 4];
    __shared__ float ws[BK][BN + 4];
    __shared__ int src_row[BM];
    qi::pdl_wait();
    const int expert = tiles[3 * blockIdx.y], row0 = tiles[3 * blockIdx.y + 1], rows = tiles[3 * blockIdx.y + 2];
    if (expert < 0 || expert >= n_experts || row0 < 0 || rows < 0 || rows > BM || row0 + rows > n_rows) return;
    const TW* we = w + (size_t)expert * N * K;
    const int tid = threadIdx.x;
    const int tx = tid % 16, ty = tid / 16;  // tx over N (16 x TN = 64), ty over M (16 x TM = 32)
    const int n0 = blockIdx.x * BN;
    if (tid < BM) src_row[tid] = tid < rows ? (gather ? order[row0 + tid] / top : row0 + tid) : -1;
    if (tid < BM && (src_row[tid] < 0 || src_row[tid] >= n_src)) src_row[tid] = -1;
    __syncthreads();

    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

    const int lrow = tid / 4;        // 0..63
    const int lk = (tid % 4) * 4;    // 0,4,8,12
    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int k = k0 + lk + i;
            float a = 0.f, b = 0.f;
            if (k < K) {
                if (lrow < BM && src_row[lrow] >= 0) a = qi::to_f32<TX>(x[(size_t)src_row[lrow] * ldx + k]);
                if (n0 + lrow < N) b = qi::to_f32<TW>(we[(size_t)(n0 + lrow) * K + k]);
            }
            if (lrow < BM) xs[lk + i][lrow] = a;
            ws[lk + i][lrow] = b;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float a[TM], b[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = xs[k][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) b[j] = ws[k][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int m = ty * TM + i;
        if (m >= rows) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int n = n0 + tx * TN + j;
            if (n < N) y[(size_t)(row0 + m) * ldy + n] = qi::from_f32<TY>(acc[i][j]);
        }
    }
}

// The same product on the tensor cores for bfloat16 operands and results (mma.sync m16n8k16, 32-bit sums, K a
// multiple of 8): a CTA of four warps takes one row tile (up to 32 sorted rows of one expert) and 64 output columns;
// the next 32 of K are requested into registers while the current ones are multiplied.
constexpr int MN = 64, MK = 32, MPAD = 8;

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__global__ void __launch_bounds__(128)
moe_gemm_mma_kernel(const qi::bf16* __restrict__ x, const qi::bf16* __restrict__ w, qi::bf16* __restrict__ y,
                    const int* __restrict__ tiles, const int* __restrict__ order, int top, int gather, int N, int K,
                    long long ldx, long long ldy, int n_src, int n_rows, int n_experts) {
    __shared__ __align__(16) qi::bf16 As[BM][MK + MPAD];
    __shared__ __align__(16) qi::bf16 Bs[MN][MK + MPAD];
    __shared__ int src_row[BM];
    qi::pdl_wait();
    const int expert = tiles[3 * blockIdx.y], row0 = tiles[3 * blockIdx.y + 1], rows = tiles[3 * blockIdx.y + 2];
    if (expert < 0 || expert >= n_experts || row0 < 0 || rows < 0 || rows > BM || row0 + rows > n_rows) return;
    const qi::bf16* we = w + (size_t)expert * N * K;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n0 = blockIdx.x * MN;
    if (tid < BM) src_row[tid] = tid < rows ? (gather ? order[row0 + tid] / top : row0 + tid) : -1;
    if (tid < BM && (src_row[tid] < 0 || src_row[tid] >= n_src)) src_row[tid] = -1;
    __syncthreads();
    const int ar = tid >> 2, ac = (tid & 3) * 8;           // this thread's 16-byte piece of the A tile (32 x 32)
    const qi::bf16* a_src = src_row[ar] >= 0 ? x + (size_t)src_row[ar] * ldx + ac : nullptr;
    const qi::bf16* b_src[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {                          // and its two pieces of the B tile (64 x 32)
        const int br = (tid >> 2) + 32 * i;
        b_src[i] = n0 + br < N ? we + (size_t)(n0 + br) * K + ac : nullptr;
    }
    auto fetch = [&](int k0, uint4& a, uint4 (&b)[2]) {
        const bool in = k0 + ac < K;
        a = (in && a_src) ? *reinterpret_cast<const uint4*>(a_src + k0) : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
        for (int i = 0; i < 2; ++i) b[i] = (in && b_src[i]) ? *reinterpret_cast<const uint4*>(b_src[i] + k0) : make_uint4(0u, 0u, 0u, 0u);
    };
    float acc[2][2][4];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 2; ++j) acc[i][j][0] = acc[i][j][1] = acc[i][j][2] = acc[i][j][3] = 0.f;
    uint4 a_reg, b_reg[2];
    fetch(0, a_reg, b_reg);
    for (int k0 = 0; k0 < K; k0 += MK) {
        __syncthreads();
        *reinterpret_cast<uint4*>(&As[ar][ac]) = a_reg;
#pragma unroll
        for (int i = 0; i < 2; ++i) *reinterpret_cast<uint4*>(&Bs[(tid >> 2) + 32 * i][ac]) = b_reg[i];
        __syncthreads();
        if (k0 + MK < K) fetch(k0 + MK, a_reg, b_reg);
#pragma unroll
        for (int kk = 0; kk < MK / 16; ++kk) {
            uint32_t a[2][4], b[2][2];
            const int c = kk * 16 + (lane & 3) * 2;
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int r = i * 16 + (lane >> 2);
                a[i][0] = *reinterpret_cast<const uint32_t*>(&As[r][c]);
                a[i][1] = *reinterpret_cast<const uint32_t*>(&As[r + 8][c]);
                a[i][2] = *reinterpret_cast<const uint32_t*>(&As[r][c + 8]);
                a[i][3] = *reinterpret_cast<const uint32_t*>(&As[r + 8][c + 8]);
            }
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int nn = warp * 16 + j * 8 + (lane >> 2);
                b[j][0] = *reinterpret_cast<const uint32_t*>(&Bs[nn][c]);
                b[j][1] = *reinterpret_cast<const uint32_t*>(&Bs[nn][c + 8]);
            }
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int j = 0; j < 2; ++j) mma_bf16_16816(acc[i][j], a[i][0], a[i][1], a[i][2], a[i][3], b[j][0], b[j][1]);
        }
    }
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int n = n0 + warp * 16 + j * 8 + (lane & 3) * 2;
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int m = i * 16 + (lane >> 2) + 8 * half;
                if (m >= rows) continue;
                qi::bf16* dst = y + (size_t)(row0 + m) * ldy + n;
                if (n < N) dst[0] = __float2bfloat16_rn(acc[i][j][2 * half]);
                if (n + 1 < N) dst[1] = __float2bfloat16_rn(acc[i][j][2 * half + 1]);
            }
        }
}

template <typename TY, typename TO>
__global__ void __launch_bounds__(256)
moe_combine_kernel(const TY* __restrict__ y, const int* __restrict__ place, const float* __restrict__ weights,
                   const TY* __restrict__ shared, TO* __restrict__ out, int n, int top, int width) {
    qi::pdl_wait();
    const size_t total = (size_t)n * width;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / width;
        const int c = (int)(idx % width);
        float acc = 0.f;
        for (int k = 0; k < top; ++k) {
            const int pl = place[t * top + k];
            if (pl >= 0 && pl < n * top) acc = fmaf(weights[t * top + k], qi::to_f32<TY>(y[(size_t)pl * width + c]), acc);
        }
        if (shared) acc += qi::to_f32<TY>(shared[idx]);
        out[idx] = qi::from_f32<TO>(acc);
    }
}

// out[i] = x[order[i] / top]: the tokens' rows in the experts' order.
template <typename T>
__global__ void __launch_bounds__(256)
moe_gather_kernel(const T* __restrict__ x, const int* __restrict__ order, int top, T* __restrict__ out, int n_pairs, int n_src, int K) {
    qi::pdl_wait();
    const size_t total = (size_t)n_pairs * K;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t i = idx / K;
        const int src = order[i] / top;
        out[idx] = (src >= 0 && src < n_src) ? x[(size_t)src * K + idx % K] : qi::from_f32<T>(0.f);
    }
}

}  // namespace

extern "C" int qi_moe_gather(const void* x, int dtype, const int* order, int top, void* out, int n_pairs, int n_src, int K,
                             cudaStream_t stream) {
    QI_REQUIRE(n_pairs >= 0 && n_src >= 0 && K > 0 && top > 0, "moe_gather: bad sizes");
    if (n_pairs == 0) return 0;
    size_t blocks = ((size_t)n_pairs * K + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    QI_DISPATCH_DTYPE(dtype, T, {
        qi::launch(moe_gather_kernel<T>, dim3((unsigned)blocks), dim3(256), 0, stream, (const T*)x, order, top, (T*)out, n_pairs, n_src, K);
    });
    return qi::check_launch("moe_gather");
}

extern "C" int qi_gemm_bf16_plan(int M, int N, int K, int allow_split, int* swap, int* bn, int* splits);
extern "C" int qi_gemm_bf16(const void* x, const void* w, void* out, int out_dtype, int M, int N, int K, int swap, int bn,
                            int splits, int epilogue, void* workspace, int* status, cudaStream_t stream);

// Every expert's rows through the dense tensor-core product, one launch an expert: x [pairs, K] in the experts' order,
// w [E, N, K], y [pairs, N], all bfloat16; bounds (HOST memory) [E + 1]: expert e owns rows bounds[e] .. bounds[e + 1] - 1.
// An expert's few hundred rows make fewer CTAs than the GPU has SMs, so the launches are dealt out over four streams
// (the caller's and three of this library's, forked from it and joined to it by events) and run side by side; every
// launch computes what it would alone. A stream that is being captured keeps all launches to itself.
extern "C" int qi_moe_gemm_by_expert(const void* x, const void* w, void* y, const int* bounds, int E, int N, int K, int* status,
                                     cudaStream_t stream) {
    QI_REQUIRE(E > 0 && N > 0 && K > 0 && K % 8 == 0 && N % 8 == 0, "moe_gemm_by_expert: bad sizes E=%d N=%d K=%d", E, N, K);
    constexpr int kSide = 3;
    static cudaStream_t side[kSide];
    static cudaEvent_t fork_ev, join_ev[kSide];
    static int side_state = 0;      // 0: not made yet, 1: ready, -1: could not be made (one stream then)
    cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(stream, &capturing) != cudaSuccess) capturing = cudaStreamCaptureStatusActive;
    if (side_state == 0) {
        bool ok = cudaEventCreateWithFlags(&fork_ev, cudaEventDisableTiming) == cudaSuccess;
        for (int i = 0; i < kSide && ok; ++i)
            ok = cudaStreamCreateWithFlags(&side[i], cudaStreamNonBlocking) == cudaSuccess &&
                 cudaEventCreateWithFlags(&join_ev[i], cudaEventDisableTiming) == cudaSuccess;
        side_state = ok ? 1 : -1;
    }
    int busy = 0;
    for (int e = 0; e < E; ++e) busy += bounds[e + 1] > bounds[e];
    const bool fan = side_state == 1 && capturing == cudaStreamCaptureStatusNone && busy > 1;
    if (fan) {
        if (cudaEventRecord(fork_ev, stream) != cudaSuccess) return qi::fail("moe_gemm_by_expert: cannot record an event");
        for (int i = 0; i < kSide; ++i)
            if (cudaStreamWaitEvent(side[i], fork_ev, 0) != cudaSuccess) return qi::fail("moe_gemm_by_expert: cannot fork a stream");
    }
    int rc = 0, launched = 0;
    for (int e = 0; e < E && !rc; ++e) {
        const int a = bounds[e], M = bounds[e + 1] - a;
        if (a < 0 || M < 0) {
            rc = qi::fail("moe_gemm_by_expert: the experts' bounds do not ascend");
            break;
        }
        if (M == 0) continue;
        int swap, bn, splits;
        qi_gemm_bf16_plan(M, N, K, 0, &swap, &bn, &splits);
        const int lane = fan ? launched % (kSide + 1) : 0;
        rc = qi_gemm_bf16((const qi::bf16*)x + (size_t)a * K, (const qi::bf16*)w + (size_t)e * N * K, (qi::bf16*)y + (size_t)a * N,
                          qi::kBF16, M, N, K, swap, bn, 1, 0, nullptr, status, lane ? side[lane - 1] : stream);
        ++launched;
    }
    if (fan) {    // joined also after a refusal, so that nothing of the side streams outlives the call's place in the stream
        for (int i = 0; i < kSide; ++i)
            if (cudaEventRecord(join_ev[i], side[i]) != cudaSuccess || cudaStreamWaitEvent(stream, join_ev[i], 0) != cudaSuccess)
                return qi::fail("moe_gemm_by_expert: cannot join a stream");
    }
    return rc;
}

extern "C" int qi_moe_tile_rows() { return BM; }

// logits float32 [n, E]; correction float32 [E] or null; ids int32 [n, top]; weights float32 [n, top].
extern "C" int qi_moe_route(const float* logits, const float* correction, int* ids, float* weights, int n, int E, int top,
                            float scale, cudaStream_t stream) {
    QI_REQUIRE(n >= 0 && E > 0 && top > 0 && top <= E, "moe_route: bad sizes n=%d experts=%d top=%d", n, E, top);
    QI_REQUIRE(E <= 32 * kMaxPerLane, "moe_route: %d experts are above this kernel's %d", E, 32 * kMaxPerLane);
    if (n == 0) return 0;
    qi::launch(moe_route_kernel, dim3((n + 3) / 4), dim3(128), 0, stream, logits, correction, ids, weights, n, E, top, scale);
    return qi::check_launch("moe_route");
}

// ids int32 [n_pairs]; offsets int32 [E + 1]; order, place int32 [n_pairs]; tiles int32 [max_tiles, 3] with
// max_tiles >= n_pairs / tile + E.
extern "C" int qi_moe_group(const int* ids, int n_pairs, int E, int tile, int max_tiles, int* offsets, int* order, int* place,
                            int* tiles, cudaStream_t stream) {
    QI_REQUIRE(n_pairs >= 0 && E > 0 && tile > 0, "moe_group: bad sizes");
    QI_REQUIRE(max_tiles >= n_pairs / tile + E || max_tiles >= n_pairs, "moe_group: the tile list is too short");
    QI_REQUIRE(E <= 4096, "moe_group: too many experts");
    qi::launch(moe_group_kernel, dim3(1), dim3(1024), sizeof(int) * (3 * (size_t)E + 2), stream, ids, n_pairs, E, tile, max_tiles,
               offsets, order, place, tiles);
    return qi::check_launch("moe_group");
}

// x rows of K (ldx apart); w [E, N, K]; y [n_rows, N] (ldy apart); tiles as moe_group wrote them with tile = qi_moe_tile_rows().
// n_src: rows of x; n_rows: rows of y (the number of (token, choice) pairs); E: experts. Tiles or source rows outside these are skipped.
extern "C" int qi_moe_gemm(const void* x, int x_dtype, const void* w, int w_dtype, void* y, int y_dtype, const int* tiles,
                           int max_tiles, const int* order, int top, int gather, int N, int K, long long ldx, long long ldy,
                           int n_src, int n_rows, int E, cudaStream_t stream) {
    QI_REQUIRE(max_tiles >= 0 && N > 0 && K > 0 && top > 0, "moe_gemm: bad sizes");
    QI_REQUIRE(ldx >= K && ldy >= N, "moe_gemm: a leading dimension is smaller than its row");
    QI_REQUIRE(max_tiles <= 65535, "moe_gemm: %d row tiles are too many for one launch", max_tiles);
    if (max_tiles == 0) return 0;
    if (x_dtype == qi::kBF16 && w_dtype == qi::kBF16 && y_dtype == qi::kBF16 && K % 8 == 0 && ldx % 8 == 0) {
        qi::launch(moe_gemm_mma_kernel, dim3((N + MN - 1) / MN, max_tiles), dim3(128), 0, stream, (const qi::bf16*)x,
                   (const qi::bf16*)w, (qi::bf16*)y, tiles, order, top, gather, N, K, ldx, ldy, n_src, n_rows, E);
        return qi::check_launch("moe_gemm_mma");
    }
    const dim3 grid((N + BN - 1) / BN, max_tiles), block(256);
    QI_DISPATCH_DTYPE(x_dtype, TX, {
        QI_DISPATCH_DTYPE(w_dtype, TW, {
            QI_DISPATCH_DTYPE(y_dtype, TY, {
                qi::launch(moe_gemm_kernel<TX, TW, TY>, grid, block, 0, stream, (const TX*)x, (const TW*)w, (TY*)y, tiles, order, top,
                           gather, N, K, ldx, ldy, n_src, n_rows, E);
            });
        });
    });
    return qi::check_launch("moe_gemm");
}

// y [n * top, width] in y_dtype (sorted rows); place int32 [n, top]; weights float32 [n, top]; shared [n, width] in y_dtype or null.
extern "C" int qi_moe_combine(const void* y, int y_dtype, const int* place, const float* weights, const void* shared, void* out,
                              int out_dtype, int n, int top, int width, cudaStream_t stream) {
    QI_REQUIRE(n >= 0 && top > 0 && width > 0, "moe_combine: bad sizes");
    if (n == 0) return 0;
    size_t blocks = ((size_t)n * width + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    QI_DISPATCH_DTYPE(y_dtype, TY, {
        QI_DISPATCH_DTYPE(out_dtype, TO, {
            qi::launch(moe_combine_kernel<TY, TO>, dim3((unsigned)blocks), dim3(256), 0, stream, (const TY*)y, place, weights,
                       (const TY*)shared, (TO*)out, n, top, width);
        });
    });
    return qi::check_launch("moe_combine");
}
