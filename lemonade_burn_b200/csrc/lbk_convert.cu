// lb-convert's per-tensor work on the device (crates/lb-convert/src/main.rs:62-87): bf16 (or f32)
// master weights -> absmean scale -> ternary values -> packed rows, with the counts of -1/0/+1 and
// the sha256 of the int8 ternary array that the converter's --check compares with torch
// (main.rs:141-170, scripts/hf_reference.py:41-58).
//
//   mean  = (f32)(sum_f64 |w| / n)            lb-ternary/src/pack.rs:135-138
//   scale = 1 / max(mean, 1e-5)               pack.rs:131
//   t     = clamp(round_ties_even(w * scale), -1, 1)   pack.rs:140-142
//   byte j of block b: bits 2k..2k+1 = t + 1 of column b*128 + k*32 + j; padding columns hold code 1 (pack.rs:88-103)
//
// All tensors of a call go through two launches (absmean, then ternarise + pack); a tensor owns a
// range of blocks in each. The f64 sum is taken as a fixed tree (per thread, per warp, per block, then over the blocks),
// not left to right as the reference's iterator does. For weights that come from bf16 (8
// significant bits each) every partial sum is exact in f64 up to millions of terms, so the order
// does not matter; for arbitrary f32 inputs the two sums can differ in the last bits of the f64,
// which moves the f32 mean only when it sits on a rounding boundary.
#include <algorithm>
#include <vector>

#include "lbk_internal.cuh"

namespace lbk {

namespace {

constexpr int kCvThreads = 256;
constexpr int kCvPartials = 1024;  // at most this many blocks (and partial sums) in the absmean pass

__device__ __forceinline__ float bf16_bits_to_f32(uint32_t b) { return __uint_as_float(b << 16); }

template <bool BF16>
__device__ __forceinline__ float load_weight(const void *src, size_t i) {
    if (BF16) return bf16_bits_to_f32(static_cast<const uint16_t *>(src)[i]);
    return static_cast<const float *>(src)[i];
}

// sum |w| in f64: partial[block]; the block that finishes last folds the partial sums (always in
// index order, whichever block that is) and writes scale = 1 / max((f32)(sum / n), 1e-5).
// One tensor of a batched launch: its buffers and the ranges of blocks that work on it in the two passes.
struct CvDev {
    const void *src;
    uint8_t *packed;
    unsigned long long rows, cols;
    unsigned a0, a1;  // blocks [a0, a1) of the absmean launch
    unsigned t0, t1;  // blocks [t0, t1) of the ternarise launch
};

// the tensor whose block range holds `block` (ranges are consecutive and non-empty)
template <bool SECOND>
__device__ __forceinline__ int find_item(const CvDev *__restrict__ items, int n, unsigned block) {
    int lo = 0, hi = n - 1;
    while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        const unsigned end = SECOND ? items[mid].t1 : items[mid].a1;
        if (block < end) hi = mid;
        else lo = mid + 1;
    }
    return lo;
}

template <bool BF16>
__global__ void __launch_bounds__(kCvThreads) absmean_partial_kernel(const CvDev *__restrict__ items, int n_items, double *__restrict__ partials,
                                                                    unsigned *__restrict__ tickets, float *__restrict__ scales) {
    __shared__ double s_red[kCvThreads / 32];
    __shared__ bool s_last;
    const int item = find_item<false>(items, n_items, blockIdx.x);
    const CvDev it = items[item];
    const void *src = it.src;
    const size_t n = it.rows * it.cols;
    const unsigned block = blockIdx.x - it.a0, n_blocks = it.a1 - it.a0;
    double *partial = partials + static_cast<size_t>(item) * kCvPartials;
    unsigned *ticket = tickets + item;
    float *scale_out = scales + item;
    constexpr int V = BF16 ? 8 : 4;  // elements per 16-byte load
    const size_t tid = static_cast<size_t>(block) * kCvThreads + threadIdx.x, stride = static_cast<size_t>(n_blocks) * kCvThreads;
    const size_t nv = (reinterpret_cast<uintptr_t>(src) & 15) == 0 ? n / V : 0;
    double s = 0.0;
    auto add16 = [&](const uint4 &v) {
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            if (BF16) {
                s += fabs(static_cast<double>(bf16_bits_to_f32(w[e] & 0xffffu)));
                s += fabs(static_cast<double>(bf16_bits_to_f32(w[e] >> 16)));
            } else {
                s += fabs(static_cast<double>(__uint_as_float(w[e])));
            }
        }
    };
    size_t i = tid;
    for (; i + 3 * stride < nv; i += 4 * stride) {  // four loads in flight per thread
        const uint4 v0 = __ldg(static_cast<const uint4 *>(src) + i), v1 = __ldg(static_cast<const uint4 *>(src) + i + stride),
                    v2 = __ldg(static_cast<const uint4 *>(src) + i + 2 * stride), v3 = __ldg(static_cast<const uint4 *>(src) + i + 3 * stride);
        add16(v0);
        add16(v1);
        add16(v2);
        add16(v3);
    }
    for (; i < nv; i += stride) add16(__ldg(static_cast<const uint4 *>(src) + i));
    for (size_t i = nv * V + tid; i < n; i += stride) s += fabs(static_cast<double>(load_weight<BF16>(src, i)));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
        double t = 0.0;
#pragma unroll
        for (int w = 0; w < kCvThreads / 32; ++w) t += s_red[w];
        partial[block] = t;
        __threadfence();
        s_last = atomicAdd(ticket, 1u) == n_blocks - 1;
    }
    __syncthreads();
    if (!s_last || threadIdx.x >= 32) return;
    __threadfence();
    double t = 0.0;
    for (unsigned i = threadIdx.x; i < n_blocks; i += 32) t += __ldcg(partial + i);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (threadIdx.x == 0) {
        const float mean = static_cast<float>(t / static_cast<double>(n));
        *scale_out = __fdiv_rn(1.0f, fmaxf(mean, 1e-5f));
        *ticket = 0u;
    }
}

// clamp(round_ties_even(x), -1, 1) + 1 for x = w * scale: +1 exactly when x > 0.5 (0.5 itself rounds to
// the even 0), -1 exactly when x < -0.5; a NaN fails both comparisons and becomes 0, as the reference's
// cast to i8 makes it.
__device__ __forceinline__ uint32_t ternary_code(float w, float scale) {
    const float x = __fmul_rn(w, scale);
    return 1u + static_cast<uint32_t>(x > 0.5f) - static_cast<uint32_t>(x < -0.5f);
}

// Eight lanes share a 128-weight block: lane q of them owns bytes 4q..4q+3, i.e. columns
// k*32 + 4q .. 4q+3 for k = 0..3, so a warp reads whole 32-byte sectors and writes 128 bytes.
template <bool BF16, typename Index>
__device__ __forceinline__ void ternarize_pack_body(const void *__restrict__ src, size_t rows, size_t cols, float scale, uint8_t *__restrict__ packed,
                                                    unsigned long long *__restrict__ counts, unsigned block, unsigned n_blocks) {
    const size_t bpr = (cols + 127) / 128, items = rows * bpr * 8;
    const bool vec = (cols & 3) == 0 && (reinterpret_cast<uintptr_t>(src) & 15) == 0;
    unsigned n_real = 0u, n_fields = 0u, n_code1 = 0u, n_code2 = 0u;
    for (size_t it = static_cast<size_t>(block) * kCvThreads + threadIdx.x; it < items; it += static_cast<size_t>(n_blocks) * kCvThreads) {
        const Index gi = static_cast<Index>(it >> 3), ri = gi / static_cast<Index>(bpr);  // 32-bit division where the sizes allow
        const size_t row = ri, blk = gi - ri * static_cast<Index>(bpr);
        const int j0 = static_cast<int>(it & 7) * 4;
        uint32_t out = 0u;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const size_t col0 = blk * 128 + k * 32 + j0;
            float w[4];
            bool have[4];
            if (vec) {
                const bool in = col0 < cols;  // cols % 4 == 0: the four columns are inside or outside together
                have[0] = have[1] = have[2] = have[3] = in;
                if (in) {
                    if (BF16) {
                        const uint2 v = __ldg(reinterpret_cast<const uint2 *>(static_cast<const uint16_t *>(src) + row * cols + col0));
                        w[0] = bf16_bits_to_f32(v.x & 0xffffu);
                        w[1] = bf16_bits_to_f32(v.x >> 16);
                        w[2] = bf16_bits_to_f32(v.y & 0xffffu);
                        w[3] = bf16_bits_to_f32(v.y >> 16);
                    } else {
                        const float4 v = __ldg(reinterpret_cast<const float4 *>(static_cast<const float *>(src) + row * cols + col0));
                        w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w;
                    }
                }
            } else {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    have[e] = col0 + e < cols;
                    if (have[e]) w[e] = load_weight<BF16>(src, row * cols + col0 + e);
                }
            }
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                uint32_t code = 1u;  // a padding column is a zero weight
                if (have[e]) {
                    code = ternary_code(w[e], scale);
                    n_real++;
                }
                out |= code << (8 * e + 2 * k);
            }
        }
        reinterpret_cast<uint32_t *>(packed)[it] = out;  // byte offset g*32 + j0
        // per 2-bit field: 00 = -1, 01 = 0, 10 = +1; padding fields are 01 as well and come off below
        n_fields += 16u;
        n_code1 += __popc(out & 0x55555555u);
        n_code2 += __popc(out & 0xaaaaaaaau);
    }
    const unsigned zeros = n_code1 - (n_fields - n_real);
    const unsigned cnt[3] = {n_real - zeros - n_code2, zeros, n_code2};
    // one global atomic per block and value: thousands of warps adding to the same three words would queue up in the L2
    __shared__ unsigned s_cnt[3];
    if (threadIdx.x < 3) s_cnt[threadIdx.x] = 0u;
    __syncthreads();
#pragma unroll
    for (int c = 0; c < 3; ++c) {
        unsigned v = cnt[c];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if ((threadIdx.x & 31) == 0 && v) atomicAdd(&s_cnt[c], v);
    }
    __syncthreads();
    if (threadIdx.x < 3 && s_cnt[threadIdx.x]) atomicAdd(counts + threadIdx.x, static_cast<unsigned long long>(s_cnt[threadIdx.x]));
}

template <bool BF16>
__global__ void __launch_bounds__(kCvThreads) ternarize_pack_kernel(const CvDev *__restrict__ items, int n_items, const float *__restrict__ scales,
                                                                   unsigned long long *__restrict__ counts) {
    const int item = find_item<true>(items, n_items, blockIdx.x);
    const CvDev it = items[item];
    const float scale = scales[item];
    const unsigned block = blockIdx.x - it.t0, n_blocks = it.t1 - it.t0;
    const unsigned long long pack_items = it.rows * ((it.cols + 127) / 128) * 8;
    if (pack_items < (1ull << 32))  // 32-bit division where the sizes allow
        ternarize_pack_body<BF16, uint32_t>(it.src, it.rows, it.cols, scale, it.packed, counts + 3 * item, block, n_blocks);
    else
        ternarize_pack_body<BF16, size_t>(it.src, it.rows, it.cols, scale, it.packed, counts + 3 * item, block, n_blocks);
}

// ---- sha256 of the ternary int8 array (row-major [rows][cols], one byte per weight: 0xff, 0, 1) ----
// FIPS 180-4. The digest of a message is a chain over its 64-byte blocks, so one tensor is one
// thread's work (lane 0 of a warp; lanes 0..15 rebuild the message words from the packed rows);
// the tensors of a model hash side by side, one warp each.
struct ShaItem {
    const uint8_t *packed;
    unsigned long long rows, cols;
};

__constant__ uint32_t kSha256K[64] = {
    0x428a2f98u, 0x71374491u, 0xb5c0fbcfu, 0xe9b5dba5u, 0x3956c25bu, 0x59f111f1u, 0x923f82a4u, 0xab1c5ed5u, 0xd807aa98u, 0x12835b01u, 0x243185beu,
    0x550c7dc3u, 0x72be5d74u, 0x80deb1feu, 0x9bdc06a7u, 0xc19bf174u, 0xe49b69c1u, 0xefbe4786u, 0x0fc19dc6u, 0x240ca1ccu, 0x2de92c6fu, 0x4a7484aau,
    0x5cb0a9dcu, 0x76f988dau, 0x983e5152u, 0xa831c66du, 0xb00327c8u, 0xbf597fc7u, 0xc6e00bf3u, 0xd5a79147u, 0x06ca6351u, 0x14292967u, 0x27b70a85u,
    0x2e1b2138u, 0x4d2c6dfcu, 0x53380d13u, 0x650a7354u, 0x766a0abbu, 0x81c2c92eu, 0x92722c85u, 0xa2bfe8a1u, 0xa81a664bu, 0xc24b8b70u, 0xc76c51a3u,
    0xd192e819u, 0xd6990624u, 0xf40e3585u, 0x106aa070u, 0x19a4c116u, 0x1e376c08u, 0x2748774cu, 0x34b0bcb5u, 0x391c0cb3u, 0x4ed8aa4au, 0x5b9cca4fu,
    0x682e6ff3u, 0x748f82eeu, 0x78a5636fu, 0x84c87814u, 0x8cc70208u, 0x90befffau, 0xa4506cebu, 0xbef9a3f7u, 0xc67178f2u};

__device__ __forceinline__ uint32_t rotr(uint32_t x, int n) { return __funnelshift_r(x, x, n); }

__device__ void sha256_compress(uint32_t (&h)[8], const uint32_t *block /* 16 big-endian words */) {
    uint32_t w[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) w[i] = block[i];
    uint32_t a = h[0], b = h[1], c = h[2], d = h[3], e = h[4], f = h[5], g = h[6], hh = h[7];
#pragma unroll
    for (int t = 0; t < 64; ++t) {
        if (t >= 16) {
            const uint32_t w15 = w[(t + 1) & 15], w2 = w[(t + 14) & 15];
            const uint32_t s0 = rotr(w15, 7) ^ rotr(w15, 18) ^ (w15 >> 3), s1 = rotr(w2, 17) ^ rotr(w2, 19) ^ (w2 >> 10);
            w[t & 15] += s0 + w[(t + 9) & 15] + s1;
        }
        const uint32_t t1 = hh + (rotr(e, 6) ^ rotr(e, 11) ^ rotr(e, 25)) + ((e & f) ^ (~e & g)) + kSha256K[t] + w[t & 15];
        const uint32_t t2 = (rotr(a, 2) ^ rotr(a, 13) ^ rotr(a, 22)) + ((a & b) ^ (a & c) ^ (b & c));
        hh = g; g = f; f = e; e = d + t1;
        d = c; c = b; b = a; a = t1 + t2;
    }
    h[0] += a; h[1] += b; h[2] += c; h[3] += d; h[4] += e; h[5] += f; h[6] += g; h[7] += hh;
}

__global__ void __launch_bounds__(32) sha256_ternary_kernel(const ShaItem *__restrict__ items, uint32_t *__restrict__ digests /* [n][8] */) {
    __shared__ uint32_t s_block[16];
    const ShaItem item = items[blockIdx.x];
    const int lane = threadIdx.x;
    const unsigned long long len = item.rows * item.cols, n_blocks = (len + 9 + 63) / 64;
    const unsigned long long rb = (item.cols + 127) / 128 * 32;
    uint32_t h[8] = {0x6a09e667u, 0xbb67ae85u, 0x3c6ef372u, 0xa54ff53au, 0x510e527fu, 0x9b05688cu, 0x1f83d9abu, 0x5be0cd19u};
    // lane l < 16 builds word l of every block: message bytes 64*b + 4*l .. +3. Its (row, col) moves on by 64 per block.
    unsigned long long pos = static_cast<unsigned long long>(lane) * 4, row = pos / item.cols, col = pos - row * item.cols;
    for (unsigned long long b = 0; b < n_blocks; ++b) {
        if (lane < 16) {
            uint32_t word = 0u;
            unsigned long long r = row, c = col;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const unsigned long long p = pos + e;
                uint32_t byte = 0u;
                if (p < len) {
                    const uint32_t code = (item.packed[r * rb + (c >> 7) * 32 + (c & 31)] >> (2 * ((c >> 5) & 3))) & 3u;
                    byte = code == 0u ? 0xffu : code - 1u;  // the i8 values -1, 0, 1
                    if (++c == item.cols) {
                        c = 0;
                        ++r;
                    }
                } else if (p == len) {
                    byte = 0x80u;
                } else if (b + 1 == n_blocks && (p & 63) >= 56) {
                    byte = static_cast<uint32_t>(((len * 8) >> (8 * (63 - (p & 63)))) & 0xffu);  // the bit length, big endian
                }
                word = (word << 8) | byte;
            }
            s_block[lane] = word;
            pos += 64;
            col += 64;
            while (col >= item.cols && row < item.rows) {  // stops once past the end, where (row, col) is no longer used
                col -= item.cols;
                ++row;
            }
        }
        __syncwarp();
        if (lane == 0) sha256_compress(h, s_block);
        __syncwarp();
    }
    if (lane == 0) {
#pragma unroll
        for (int i = 0; i < 8; ++i) digests[static_cast<size_t>(blockIdx.x) * 8 + i] = h[i];
    }
}

}  // namespace

}  // namespace lbk

using namespace lbk;

extern "C" {

int lbk_convert_bitlinear(lbk_ctx *c, const lbk_convert_item *items, size_t n, int src_dtype, float *scales_out, uint64_t *counts_out,
                          uint8_t *sha256_out, void *stream) {
    if (!c) return fail(LBK_ERR_INVALID, "lbk_convert_bitlinear: context is null");
    Ctx *ctx = reinterpret_cast<Ctx *>(c);
    if (n == 0) return LBK_OK;
    if (!items || !scales_out) return fail(LBK_ERR_INVALID, "lbk_convert_bitlinear: null argument");
    if (src_dtype != LBK_DTYPE_F32 && src_dtype != LBK_DTYPE_BF16) return fail(LBK_ERR_INVALID, "source dtype must be LBK_DTYPE_F32 or LBK_DTYPE_BF16");
    const bool bf16 = src_dtype == LBK_DTYPE_BF16;
    for (size_t i = 0; i < n; ++i) {
        const lbk_convert_item &it = items[i];
        if (!it.src_dev || !it.packed_dev || it.rows == 0 || it.cols == 0) return fail(LBK_ERR_INVALID, "tensor %zu: null buffer or empty shape", i);
        if (reinterpret_cast<uintptr_t>(it.src_dev) % (bf16 ? 2 : 4) || reinterpret_cast<uintptr_t>(it.packed_dev) % 4)
            return fail(LBK_ERR_INVALID, "tensor %zu: misaligned buffer", i);
    }
    LBK_CUDA(cudaSetDevice(ctx->device));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    struct Work {
        double *partial = nullptr;
        float *scales = nullptr;
        unsigned long long *counts = nullptr;
        ShaItem *sha_items = nullptr;
        uint32_t *digests = nullptr;
        CvDev *table = nullptr;
        ~Work() {
            cudaFree(table);
            cudaFree(partial);
            cudaFree(scales);
            cudaFree(counts);
            cudaFree(sha_items);
            cudaFree(digests);
        }
    } wk;
    LBK_CUDA(cudaMalloc(&wk.partial, n * kCvPartials * sizeof(double)));
    LBK_CUDA(cudaMalloc(&wk.scales, n * sizeof(float)));
    LBK_CUDA(cudaMalloc(&wk.counts, n * 4 * sizeof(unsigned long long)));  // [n][3] counts, then n tickets
    LBK_CUDA(cudaMemsetAsync(wk.counts, 0, n * 4 * sizeof(unsigned long long), st));
    unsigned *tickets = reinterpret_cast<unsigned *>(wk.counts + 3 * n);
    // two launches for the whole batch: every tensor gets a range of blocks in each
    std::vector<CvDev> table(n);
    unsigned a_blocks = 0, t_blocks = 0;
    for (size_t i = 0; i < n; ++i) {
        const lbk_convert_item &it = items[i];
        const size_t elems = it.rows * it.cols;
        const size_t per_block = static_cast<size_t>(kCvThreads) * 32;
        const unsigned blocks_a = static_cast<unsigned>(std::min<size_t>(std::min<size_t>(kCvPartials, static_cast<size_t>(ctx->sm_count) * 6), (elems + per_block - 1) / per_block));
        const size_t pack_items = it.rows * ((it.cols + 127) / 128) * 8;
        const unsigned blocks_t = static_cast<unsigned>(std::min<size_t>(static_cast<size_t>(ctx->sm_count) * 8, (pack_items + kCvThreads * 4 - 1) / (kCvThreads * 4)));
        table[i] = CvDev{it.src_dev, it.packed_dev, it.rows, it.cols, a_blocks, a_blocks + blocks_a, t_blocks, t_blocks + blocks_t};
        a_blocks += blocks_a;
        t_blocks += blocks_t;
    }
    LBK_CUDA(cudaMalloc(&wk.table, n * sizeof(CvDev)));
    LBK_CUDA(cudaMemcpyAsync(wk.table, table.data(), n * sizeof(CvDev), cudaMemcpyHostToDevice, st));
    LBK_CUDA(cudaStreamSynchronize(st));  // `table` is pageable
    if (bf16) {
        absmean_partial_kernel<true><<<a_blocks, kCvThreads, 0, st>>>(wk.table, static_cast<int>(n), wk.partial, tickets, wk.scales);
        ternarize_pack_kernel<true><<<t_blocks, kCvThreads, 0, st>>>(wk.table, static_cast<int>(n), wk.scales, wk.counts);
    } else {
        absmean_partial_kernel<false><<<a_blocks, kCvThreads, 0, st>>>(wk.table, static_cast<int>(n), wk.partial, tickets, wk.scales);
        ternarize_pack_kernel<false><<<t_blocks, kCvThreads, 0, st>>>(wk.table, static_cast<int>(n), wk.scales, wk.counts);
    }
    ctx->launches += 2;
    LBK_CUDA(cudaGetLastError());
    std::vector<uint32_t> digests;
    if (sha256_out) {
        std::vector<ShaItem> sh(n);
        for (size_t i = 0; i < n; ++i) sh[i] = ShaItem{items[i].packed_dev, items[i].rows, items[i].cols};
        LBK_CUDA(cudaMalloc(&wk.sha_items, n * sizeof(ShaItem)));
        LBK_CUDA(cudaMalloc(&wk.digests, n * 8 * sizeof(uint32_t)));
        LBK_CUDA(cudaMemcpyAsync(wk.sha_items, sh.data(), n * sizeof(ShaItem), cudaMemcpyHostToDevice, st));
        LBK_CUDA(cudaStreamSynchronize(st));  // `sh` goes away
        sha256_ternary_kernel<<<static_cast<unsigned>(n), 32, 0, st>>>(wk.sha_items, wk.digests);
        LBK_CUDA(cudaGetLastError());
        ctx->launches += 1;
        digests.resize(n * 8);
        LBK_CUDA(cudaMemcpyAsync(digests.data(), wk.digests, n * 8 * sizeof(uint32_t), cudaMemcpyDeviceToHost, st));
    }
    std::vector<unsigned long long> counts(n * 3);
    LBK_CUDA(cudaMemcpyAsync(scales_out, wk.scales, n * sizeof(float), cudaMemcpyDeviceToHost, st));
    LBK_CUDA(cudaMemcpyAsync(counts.data(), wk.counts, n * 3 * sizeof(unsigned long long), cudaMemcpyDeviceToHost, st));
    LBK_CUDA(cudaStreamSynchronize(st));
    if (counts_out)
        for (size_t i = 0; i < n * 3; ++i) counts_out[i] = counts[i];
    if (sha256_out)
        for (size_t i = 0; i < n * 8; ++i) {  // big-endian words, as the digest is written
            sha256_out[4 * i] = static_cast<uint8_t>(digests[i] >> 24);
            sha256_out[4 * i + 1] = static_cast<uint8_t>(digests[i] >> 16);
            sha256_out[4 * i + 2] = static_cast<uint8_t>(digests[i] >> 8);
            sha256_out[4 * i + 3] = static_cast<uint8_t>(digests[i]);
        }
    return LBK_OK;
}

}  // extern "C"
