// A batch of small matrix products on the tensor cores: y_b[M, N] = x_b[M, K] . w_b[N, K]^T for b < batch,
// bfloat16 operands and output, 32-bit accumulation (mma.sync m16n8k16). Product b reads x + b * sx,
// w + b * sw and writes y + b * sy (strides in elements), with row strides ldx, ldw, ldy: the per-head
// projections of an attention whose heads lie side by side in one activation row (sx = a head's width,
// ldx = the row's), each head with a matrix of its own. Both operands are read along K.
//
// A CTA computes a 64 x 64 tile with four warps of 16 rows; K advances in steps of 64 through two
// cp.async buffers; rows are padded by 16 bytes against ldmatrix bank conflicts. These products are
// small (K and N of a head's size), so the kernel is bound by its operands' traffic, not by the tensor
// pipe; what matters is that all heads run in one launch.
#include "attention_frag.cuh"

namespace {

using namespace qi_attn;
using qi::bf16;

constexpr int BM = 64, BN = 64, BK = 64;
constexpr int kStride = BK * 2 + 16;
constexpr int kChunks = BK / 8;

__device__ __forceinline__ void cp16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void zero16(uint32_t dst) {
    asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(dst), "r"(0u) : "memory");
}

__global__ void __launch_bounds__(128)
gemm_mma_batched_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w, bf16* __restrict__ y, int M, int N, int K,
                        long long ldx, long long ldw, long long ldy, long long sx, long long sw, long long sy) {
    __shared__ __align__(128) unsigned char smem[2 * (BM + BN) * kStride];
    qi::pdl_wait();
    x += (size_t)blockIdx.z * sx;
    w += (size_t)blockIdx.z * sw;
    y += (size_t)blockIdx.z * sy;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t base = smem_u32(smem);
    auto load = [&](int k0, int buf) {
        const uint32_t xs = base + buf * (BM + BN) * kStride, ws = xs + BM * kStride;
        for (int idx = threadIdx.x; idx < (BM + BN) * kChunks; idx += 128) {
            const int row = idx / kChunks, chunk = idx % kChunks;
            const int k = k0 + chunk * 8;
            if (row < BM) {
                const uint32_t dst = xs + row * kStride + (chunk << 4);
                if (m0 + row < M && k < K) cp16(dst, x + (size_t)(m0 + row) * ldx + k);
                else zero16(dst);
            } else {
                const int r = row - BM;
                const uint32_t dst = ws + r * kStride + (chunk << 4);
                if (n0 + r < N && k < K) cp16(dst, w + (size_t)(n0 + r) * ldw + k);
                else zero16(dst);
            }
        }
    };
    float acc[BN / 8][4];
#pragma unroll
    for (int j = 0; j < BN / 8; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[j][e] = 0.f;
    const int steps = (K + BK - 1) / BK;
    load(0, 0);
    asm volatile("cp.async.commit_group;" ::: "memory");
    for (int it = 0; it < steps; ++it) {
        if (it + 1 < steps) load((it + 1) * BK, (it + 1) & 1);
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 1;" ::: "memory");
        __syncthreads();
        const uint32_t xs = base + (it & 1) * (BM + BN) * kStride, ws = xs + BM * kStride;
#pragma unroll
        for (int ks = 0; ks < BK / 16; ++ks) {
            uint32_t a[4];
            ldmatrix_x4(xs + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * kStride + ((ks * 2 + (lane >> 4)) << 4), a[0], a[1], a[2], a[3]);
#pragma unroll
            for (int jp = 0; jp < BN / 16; ++jp) {
                uint32_t r0, r1, r2, r3;
                ldmatrix_x4(ws + (jp * 16 + (lane & 7) + (lane >> 4) * 8) * kStride + ((ks * 2 + ((lane >> 3) & 1)) << 4), r0, r1, r2, r3);
                mma_bf16(acc[2 * jp], a, r0, r1);
                mma_bf16(acc[2 * jp + 1], a, r2, r3);
            }
        }
        __syncthreads();
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    const int g = lane >> 2, c2 = (lane & 3) * 2;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int m = m0 + warp * 16 + g + r * 8;
        if (m >= M) continue;
        bf16* row = y + (size_t)m * ldy;
#pragma unroll
        for (int j = 0; j < BN / 8; ++j) {
            const int n = n0 + j * 8 + c2;
            if (n + 1 < N) *reinterpret_cast<__nv_bfloat162*>(row + n) = __floats2bfloat162_rn(acc[j][2 * r], acc[j][2 * r + 1]);
            else if (n < N) row[n] = __float2bfloat16_rn(acc[j][2 * r]);
        }
    }
}

}  // namespace

// 16-byte loads: K and every stride that moves an operand's row start must be a multiple of 8 elements, the
// operands' bases 16-byte aligned; 4-byte stores: ldy, sy even and y 4-byte aligned.
extern "C" int qi_gemm_mma_batched_supported(const void* x, const void* w, const void* y, int K, long long ldx, long long ldw,
                                             long long ldy, long long sx, long long sw, long long sy) {
    return K % 8 == 0 && ldx % 8 == 0 && ldw % 8 == 0 && sx % 8 == 0 && sw % 8 == 0 && ((uintptr_t)x & 15) == 0 &&
           ((uintptr_t)w & 15) == 0 && ldy % 2 == 0 && sy % 2 == 0 && ((uintptr_t)y & 3) == 0;
}

extern "C" int qi_gemm_mma_batched(const void* x, const void* w, void* y, int M, int N, int K, long long ldx, long long ldw,
                                   long long ldy, int batch, long long sx, long long sw, long long sy, cudaStream_t stream) {
    QI_REQUIRE(M >= 0 && N > 0 && K > 0 && batch > 0 && batch <= 65535, "gemm_mma_batched: bad sizes M=%d N=%d K=%d batch=%d", M, N, K, batch);
    QI_REQUIRE(qi_gemm_mma_batched_supported(x, w, y, K, ldx, ldw, ldy, sx, sw, sy), "gemm_mma_batched: operands are not aligned for 16-byte loads");
    QI_REQUIRE((M + BM - 1) / BM <= 65535, "gemm_mma_batched: M=%d is too large for one launch", M);
    if (M == 0) return 0;
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM, batch);
    qi::launch(gemm_mma_batched_kernel, grid, dim3(128), 0, stream, (const bf16*)x, (const bf16*)w, (bf16*)y, M, N, K, ldx, ldw, ldy, sx,
               sw, sy);
    return qi::check_launch("gemm_mma_batched");
}
