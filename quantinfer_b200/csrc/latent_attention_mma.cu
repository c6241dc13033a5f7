// Attention over a cached latent on the tensor cores (bfloat16 operands, 32-bit scores, softmax and sums):
// the flash form of latent_attention.cu for prompts' portions and single decode tokens alike.
//
// All heads of a token read the SAME cached rows [c | kr] of width W = R + r, and the value is the row's
// first R numbers. So the rows of a query tile are (token, head) pairs of one request, 16 x MW of them a CTA
// (MW warps of 16: eight for a step that holds portions of prompts, four for a step of single tokens), and
// one key tile in shared memory serves every head, once as the B operand of S = Q K^T (over W) and once more,
// read transposed, as the B operand of O += P V (over its first R columns). With H heads a tile of N rows
// holds N / H tokens (H <= N), or N of one token's heads (H > N, the heads then spread over grid.y). A decode
// token is a tile of H rows.
//
// Tiles are found on the device: CTA x walks the entries' lengths (q_start) until it meets the entry that
// holds its tile, so a launch needs no host-side list and can be replayed from a CUDA graph; the grid is an
// upper bound (tokens / tokens-per-tile + entries) and the CTAs beyond the last tile leave at once.
//
// Key tiles of 64 positions (32 for rows wider than 192 in CTAs of four warps, so that two share an SM) start at multiples of
// their size in the absolute position, whatever the portion: the sums of a query row are formed in the same
// order however the prompt was cut. A step of few query tiles and many keys (decode) spreads every tile's key
// tiles over grid.z; the ranges' partial sums meet in a second kernel, which also adds the sink. Rows of the tile outside
// [first visible key, last query] are zero-filled and never looked up (their pages may be free again behind
// a window); each score is masked by its own row's causal bound and window. The softmax's denominator
// takes exp(sink_h) once, at the end. Key tiles are double-buffered with cp.async; rows are padded by 16
// bytes, which keeps ldmatrix free of bank conflicts for any W that is a multiple of 16.
#include "attention_frag.cuh"

namespace {

using namespace qi_attn;
using qi::bf16;


template <int W> struct PadRows {
    static constexpr int kStride = W * 2 + 16;
    static __device__ __forceinline__ uint32_t off(int row, int chunk) { return (uint32_t)(row * kStride + (chunk << 4)); }
};

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void st_zero16(uint32_t dst) {
    asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(dst), "r"(0u) : "memory");
}

template <int W, int R, int KT, int MW>
__global__ void __launch_bounds__(32 * MW)
latent_attention_mma_kernel(const bf16* __restrict__ q, bf16* __restrict__ out, const bf16* __restrict__ cache,
                            const float* __restrict__ sink, const int* __restrict__ block_table, int max_blocks,
                            int page_size, int num_pages, const int* __restrict__ q_start,
                            const int* __restrict__ start_pos, int n_requests, int H, float scale_log2, int window,
                            int n_splits, float* __restrict__ ws_o, float* __restrict__ ws_ml, int* __restrict__ status) {
    using Addr = PadRows<W>;
    constexpr int kRows = 16 * MW, kThreads = 32 * MW;      // MW warps of 16 query rows
    constexpr int kChunks = W / 8;
    constexpr int NT = KT / 8;
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ int s_entry, s_t0;
    const uint32_t q_s = smem_u32(smem);
    const uint32_t k_s = q_s + kRows * Addr::kStride;
    constexpr uint32_t kTileBytes = KT * Addr::kStride;

    qi::pdl_wait();
    const int rpt = H < kRows ? H : kRows;      // rows of a tile per token
    const int TQ = kRows / rpt;                 // tokens of a tile
    if (threadIdx.x < 32) {
        // warp 0 walks the entries 32 at a time: each lane one entry's tile count, a prefix sum over the lanes
        const int lane = threadIdx.x;
        int c = blockIdx.x, found = -1, t0 = 0;
        for (int e0 = 0; e0 < n_requests && found < 0; e0 += 32) {
            const int e = e0 + lane;
            const int a = e < n_requests ? q_start[e] : 0;
            const int nt = e < n_requests ? (q_start[e + 1] - a + TQ - 1) / TQ : 0;
            int incl = nt;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int v = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += v;
            }
            const unsigned hit = __ballot_sync(0xffffffffu, c < incl);
            if (hit) {
                const int src = __ffs(hit) - 1;
                found = e0 + src;
                // an entry's tiles from its end: the tiles with the most keys start first, the short ones fill the tail
                const int within = c - __shfl_sync(0xffffffffu, incl - nt, src);
                t0 = __shfl_sync(0xffffffffu, a, src) + (__shfl_sync(0xffffffffu, nt, src) - 1 - within) * TQ;
            } else {
                c -= __shfl_sync(0xffffffffu, incl, 31);
            }
        }
        if (lane == 0) {
            s_entry = found;
            s_t0 = t0;
        }
    }
    __syncthreads();
    const int e = s_entry, t0 = s_t0;
    if (e < 0) return;
    const int first = q_start[e], len = q_start[e + 1] - first;
    const int ntok = min(TQ, first + len - t0);
    const int h0 = blockIdx.y * kRows;
    const int nvalid = H <= kRows ? ntok * H : min(kRows, H - h0);
    const int p_lo = start_pos[e] + (t0 - first), p_hi = p_lo + ntok - 1;
    const int key_lo = (window > 0 && p_lo - window + 1 > 0) ? p_lo - window + 1 : 0;
    const int* table = block_table + (size_t)e * max_blocks;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k_begin = key_lo / KT * KT;
    const int n_tiles = (p_hi - k_begin) / KT + 1;
    // with key ranges (grid.z, a decode step): this CTA's share of the key tiles; its rows' partial sums go to the
    // workspace and a second kernel adds the ranges. A range without tiles leaves empty partial sums.
    int it0 = 0, it1 = n_tiles;
    if (n_splits > 1) {
        const int per = (n_tiles + n_splits - 1) / n_splits;
        it0 = blockIdx.z * per;
        it1 = min(n_tiles, it0 + per);
        if (it0 >= it1) {
            for (int rho = threadIdx.x; rho < nvalid; rho += kThreads) {
                float* ml = ws_ml + (((size_t)t0 * H + h0 + rho) * n_splits + blockIdx.z) * 2;
                ml[0] = -INFINITY;
                ml[1] = 0.f;
            }
            return;
        }
    }

    // the query rows: contiguous in memory from row t0 * H + h0
    const bf16* q_rows = q + ((size_t)t0 * H + h0) * W;
    for (int idx = threadIdx.x; idx < kRows * kChunks; idx += kThreads) {
        const int row = idx / kChunks, chunk = idx % kChunks;
        const uint32_t dst = q_s + Addr::off(row, chunk);
        if (row < nvalid) cp_async16(dst, q_rows + (size_t)row * W + chunk * 8);
        else st_zero16(dst);
    }
    bool bad_page = false;
    auto load_keys = [&](int k0, int buf) {
        const uint32_t base = k_s + buf * kTileBytes;
        for (int idx = threadIdx.x; idx < KT * kChunks; idx += kThreads) {
            const int row = idx / kChunks, chunk = idx % kChunks;
            const int j = k0 + row;
            const uint32_t dst = base + Addr::off(row, chunk);
            const bf16* src = nullptr;
            if (j >= key_lo && j <= p_hi) {
                const int page = table[j / page_size];
                if (page < 0 || page >= num_pages) bad_page = true;
                else src = cache + ((size_t)page * page_size + j % page_size) * W + chunk * 8;
            }
            if (src) cp_async16(dst, src);
            else st_zero16(dst);
        }
    };
    load_keys(k_begin + it0 * KT, 0);
    cp_commit();

    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    float o[R / 8][4];
#pragma unroll
    for (int n = 0; n < R / 8; ++n)
#pragma unroll
        for (int x = 0; x < 4; ++x) o[n][x] = 0.f;
    const int row0 = warp * 16;
    const bool active = row0 < nvalid;
    const int g = lane >> 2;
    int p_row[2], lo_row[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int rho = row0 + g + r * 8;
        p_row[r] = rho < nvalid ? p_lo + rho / rpt : -1;       // -1: no key passes `key <= p_row`
        lo_row[r] = window > 0 ? p_row[r] - window + 1 : 0;
    }

    for (int it = it0; it < it1; ++it) {
        const int k0 = k_begin + it * KT;
        if (it + 1 < it1) load_keys(k0 + KT, (it - it0 + 1) & 1);
        cp_commit();
        cp_wait<1>();
        __syncthreads();
        if (active) {
            const uint32_t kt = k_s + ((it - it0) & 1) * kTileBytes;
            float s[NT][4];
#pragma unroll
            for (int j = 0; j < NT; ++j)
#pragma unroll
                for (int x = 0; x < 4; ++x) s[j][x] = 0.f;
#pragma unroll 2
            for (int ks = 0; ks < W / 16; ++ks) {
                uint32_t a[4];
                ldmatrix_x4(q_s + Addr::off(row0 + (lane & 7) + ((lane >> 3) & 1) * 8, ks * 2 + (lane >> 4)), a[0], a[1], a[2], a[3]);
#pragma unroll
                for (int jp = 0; jp < NT / 2; ++jp) {
                    uint32_t r0, r1, r2, r3;
                    ldmatrix_x4(kt + Addr::off(jp * 16 + (lane & 7) + (lane >> 4) * 8, ks * 2 + ((lane >> 3) & 1)), r0, r1, r2, r3);
                    mma_bf16(s[2 * jp], a, r0, r1);
                    mma_bf16(s[2 * jp + 1], a, r2, r3);
                }
            }
#pragma unroll
            for (int j = 0; j < NT; ++j)
#pragma unroll
                for (int x = 0; x < 4; ++x) {
                    const int key = k0 + j * 8 + (lane & 3) * 2 + (x & 1);
                    const int r = x >> 1;
                    if (key > p_row[r] || key < lo_row[r]) s[j][x] = -INFINITY;
                }
            softmax_tile<R, NT>(s, m, l, o, scale_log2);
            pv_tile<R, NT, Addr>(o, s, kt, 0, lane);
        }
        __syncthreads();
    }
    cp_wait<0>();
    if (bad_page && status) atomicOr(status, qi::kStatusBadPage);
    if (!active) return;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int rho = row0 + g + r * 8;
        float sum = l[r];
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        if (rho >= nvalid) continue;
        if (n_splits > 1) {
            const size_t slot = ((size_t)t0 * H + h0 + rho) * n_splits + blockIdx.z;
            if ((lane & 3) == 0) {
                ws_ml[slot * 2] = m[r];
                ws_ml[slot * 2 + 1] = sum;
            }
            float* po = ws_o + slot * R + (lane & 3) * 2;
#pragma unroll
            for (int n = 0; n < R / 8; ++n) *reinterpret_cast<float2*>(po + n * 8) = make_float2(o[n][2 * r], o[n][2 * r + 1]);
            continue;
        }
        const int h = h0 + rho % rpt;
        const float sk = sink ? sink[h] * 1.4426950408889634f : -INFINITY;
        const float mf = fmaxf(m[r], sk);
        const float a = (m[r] == -INFINITY) ? 0.f : ex2(m[r] - mf);
        const float denom = sum * a + (sink ? ex2(sk - mf) : 0.f);
        const float f = denom > 0.f ? a / denom : 0.f;
        bf16* dst = out + ((size_t)t0 * H + h0 + rho) * R + (lane & 3) * 2;
#pragma unroll
        for (int n = 0; n < R / 8; ++n)
            *reinterpret_cast<__nv_bfloat162*>(dst + n * 8) = __floats2bfloat162_rn(o[n][2 * r] * f, o[n][2 * r + 1] * f);
    }
}

// Adds the key ranges of a row: out = sum_i o_i 2^(m_i - M) / (sum_i l_i 2^(m_i - M) + 2^(sink - M)), M the largest of
// the ranges' maxima and the sink (all in the base-2 scale of the main kernel).
template <int R>
__global__ void latent_attention_merge_kernel(const float* __restrict__ ws_o, const float* __restrict__ ws_ml,
                                              const float* __restrict__ sink, bf16* __restrict__ out, int H, int n_splits) {
    extern __shared__ float wgt[];      // [n_splits]: 2^(m_i - M) / denominator, 0 for an empty range
    __shared__ float s_red[2];
    qi::pdl_wait();
    const size_t row = blockIdx.x;
    const float sk = sink ? sink[row % H] * 1.4426950408889634f : -INFINITY;
    if (threadIdx.x < 32) {
        // one warp: lane i takes ranges i, i + 32, ...; their loads are in flight together
        const int lane = threadIdx.x;
        float M = sk;
        for (int i = lane; i < n_splits; i += 32) M = fmaxf(M, ws_ml[(row * n_splits + i) * 2]);
        M = qi::warp_max(M);
        float denom = 0.f;
        for (int i = lane; i < n_splits; i += 32) {
            const float mi = ws_ml[(row * n_splits + i) * 2];
            const float f = mi == -INFINITY ? 0.f : ex2(mi - M);
            wgt[i] = f;
            denom += f * ws_ml[(row * n_splits + i) * 2 + 1];
        }
        denom = qi::warp_sum(denom) + (sink ? ex2(sk - M) : 0.f);
        if (lane == 0) s_red[0] = denom > 0.f ? 1.0f / denom : 0.f;
    }
    __syncthreads();
    const float inv = s_red[0];
    for (int c = threadIdx.x; c < R; c += blockDim.x) {
        float acc = 0.f;
#pragma unroll 4
        for (int i = 0; i < n_splits; ++i)
            if (wgt[i] != 0.f) acc = fmaf(ws_o[(row * n_splits + i) * R + c], wgt[i], acc);   // an empty range wrote no sums
        out[row * R + c] = __float2bfloat16_rn(acc * inv);
    }
}

template <int W, int R, int MW>
int launch_mma(const void* q, void* out, const void* cache, const float* sink, const int* block_table, int max_blocks,
               int page_size, int num_pages, const int* q_start, const int* start_pos, int n_requests, int n_tokens, int H,
               float scale, int window, int n_splits, float* ws_o, float* ws_ml, int* status, cudaStream_t stream) {
    // wide rows in CTAs of four warps: shorter key tiles, so that two CTAs share an SM (a CTA of eight warps has the
    // SM to itself by its registers anyway)
    constexpr int KT = (W > 192 && MW == 4) ? 32 : 64;
    constexpr int kRows = 16 * MW, kThreads = 32 * MW;
    const size_t smem = (size_t)(kRows + 2 * KT) * PadRows<W>::kStride;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(latent_attention_mma_kernel<W, R, KT, MW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return qi::fail("latent_attention_mma: %zu bytes of shared memory were refused", smem);
        configured = true;
    }
    const int rpt = H < kRows ? H : kRows;
    const int TQ = kRows / rpt;
    const long long tiles = (long long)n_tokens / TQ + n_requests;
    QI_REQUIRE(tiles <= 0x7fffffffll, "latent_attention_mma: grid too large");
    dim3 grid((unsigned)tiles, (unsigned)((H + kRows - 1) / kRows), (unsigned)n_splits);
    qi::launch(latent_attention_mma_kernel<W, R, KT, MW>, grid, dim3(kThreads), smem, stream, (const bf16*)q, (bf16*)out, (const bf16*)cache, sink,
               block_table, max_blocks, page_size, num_pages, q_start, start_pos, n_requests, H, scale * 1.4426950408889634f, window,
               n_splits, ws_o, ws_ml, status);
    if (n_splits > 1)
        qi::launch(latent_attention_merge_kernel<R>, dim3((unsigned)((size_t)n_tokens * H)), dim3(R >= 128 ? 128 : 64), sizeof(float) * n_splits, stream,
                   (const float*)ws_o, (const float*)ws_ml, sink, (bf16*)out, H, n_splits);
    return qi::check_launch("latent_attention_mma");
}

}  // namespace

// Latent widths R in {32, 64, 128, 256} with a rotated part r in {16, 32, 64}.
extern "C" int qi_latent_attention_mma_supported(int W, int R) {
    const int r = W - R;
    return (R == 32 || R == 64 || R == 128 || R == 256) && (r == 16 || r == 32 || r == 64);
}

// Key tiles of a query tile per CTA: 64 keys, or 32 for rows wider than 192.
extern "C" int qi_latent_attention_mma_key_tile(int W) { return W > 192 ? 32 : 64; }      // (of a step of single tokens)

// n_splits > 1 cuts every query tile's keys into that many ranges over grid.z (for steps of few query tiles and many
// keys: decode); ws_o float32 [n * H, n_splits, R] and ws_ml float32 [n * H, n_splits, 2] then take the partial sums.
// q [n, H, W], out [n, H, R], cache [num_pages, page_size, W], all bfloat16; sink float32 [H] or null; q_start
// [n_requests + 1] and start_pos [n_requests] as in the step's arrays (entry e's rows are q_start[e] ..
// q_start[e + 1] - 1 at positions start_pos[e] ...).
extern "C" int qi_latent_attention_mma(const void* q, void* out, const void* cache, const float* sink, const int* block_table,
                                       int max_blocks, int page_size, int num_pages, const int* q_start, const int* start_pos,
                                       int n_requests, int n_tokens, int H, int W, int R, float scale, int window, int n_splits,
                                       float* ws_o, float* ws_ml, int* status, cudaStream_t stream) {
    QI_REQUIRE(n_splits >= 1 && n_splits <= 65535 && (n_splits == 1 || (ws_o && ws_ml)), "latent_attention_mma: bad key ranges or no workspace for them");
    QI_REQUIRE((long long)n_tokens * H <= 0x7fffffffll, "latent_attention_mma: too many rows");
    QI_REQUIRE(qi_latent_attention_mma_supported(W, R), "latent_attention_mma: a latent of %d with a rotated part of %d is not covered", R, W - R);
    QI_REQUIRE(n_tokens >= 0 && n_requests >= 0 && H > 0 && H <= 65535 * 64, "latent_attention_mma: bad sizes");
    QI_REQUIRE(page_size > 0 && max_blocks > 0 && num_pages > 0 && window >= 0, "latent_attention_mma: bad page geometry or window");
    if (n_tokens == 0 || n_requests == 0) return 0;
    // a step with portions of prompts: CTAs of eight warps (128 rows: more tokens share a key tile, and head counts
    // that do not divide 64 fill their rows better); a step of single tokens: four warps
    const bool wide = n_tokens > n_requests;
#define QI_LATENT_CASE(RR, rr)                                                                                                     \
    if (R == RR && W - R == rr)                                                                                                    \
        return wide ? launch_mma<RR + rr, RR, 8>(q, out, cache, sink, block_table, max_blocks, page_size, num_pages, q_start,      \
                                                 start_pos, n_requests, n_tokens, H, scale, window, n_splits, ws_o, ws_ml, status, \
                                                 stream)                                                                           \
                    : launch_mma<RR + rr, RR, 4>(q, out, cache, sink, block_table, max_blocks, page_size, num_pages, q_start,      \
                                                 start_pos, n_requests, n_tokens, H, scale, window, n_splits, ws_o, ws_ml, status, \
                                                 stream);
    QI_LATENT_CASE(32, 16) QI_LATENT_CASE(32, 32) QI_LATENT_CASE(32, 64)
    QI_LATENT_CASE(64, 16) QI_LATENT_CASE(64, 32) QI_LATENT_CASE(64, 64)
    QI_LATENT_CASE(128, 16) QI_LATENT_CASE(128, 32) QI_LATENT_CASE(128, 64)
    QI_LATENT_CASE(256, 16) QI_LATENT_CASE(256, 32) QI_LATENT_CASE(256, 64)
#undef QI_LATENT_CASE
    return qi::fail("latent_attention_mma: no kernel for these sizes");
}
