// Kernels that prepare memory rather than compute on it: handing cache pages to sequences, and the
// seeded fill of random weights.
#include "common.cuh"

// ------------------------------------------------------------------------------------------
// Pages handed out.  `triples` holds (slot, logical page, physical page) for every page that the
// step gives to a sequence.  One kernel writes the block table; another clears the pages in every
// plane of a group, so that a page never carries what an earlier sequence left in it: the
// tensor-core attention kernels feed whole 64-key pages into P.V with P = 0 beyond a sequence's
// length, and 0 times a stale Inf or NaN would not be 0.
__global__ void block_table_set_kernel(int* __restrict__ table, int bt_stride, int max_slots, const int* __restrict__ triples, int n) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int slot = triples[3 * i], lp = triples[3 * i + 1], page = triples[3 * i + 2];
    // checked on the host; never out of bounds
    if (!gb_check(slot, max_slots, GB_CHECK_TRIPLE) || !gb_check(lp, bt_stride, GB_CHECK_TRIPLE)) return;
    if (slot < 0 || slot >= max_slots || lp < 0 || lp >= bt_stride) return;
    table[(int64_t)slot * bt_stride + lp] = page;
}

GB_API int gb_block_table_set(int* table, int bt_stride, int max_slots, const int* triples, int n, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (bt_stride <= 0 || max_slots <= 0) GB_REFUSE("block_table_set: table of %d x %d", max_slots, bt_stride);
    block_table_set_kernel<<<ceil_div(n, 128), 128, 0, stream>>>(table, bt_stride, max_slots, triples, n);
    GB_CHECK_LAUNCH("block_table_set");
    return 0;
}

__global__ void zero_pages_kernel(unsigned char* __restrict__ base, int64_t plane_stride, int64_t page_bytes, int n_pages,
                                  const int* __restrict__ triples) {
    const int page = triples[3 * blockIdx.x + 2];
    if (!gb_check(page, n_pages, GB_CHECK_TRIPLE) || page < 0 || page >= n_pages) return;
    uint4* dst = reinterpret_cast<uint4*>(base + (int64_t)blockIdx.y * plane_stride + (int64_t)page * page_bytes);
    const int64_t n16 = page_bytes >> 4;
    for (int64_t i = threadIdx.x; i < n16; i += blockDim.x) dst[i] = make_uint4(0u, 0u, 0u, 0u);
}

// base: [planes][n_pages][page_bytes]; clears page triples[3 i + 2] of every plane, i < n
GB_API int gb_zero_pages(void* base, int64_t plane_stride, int planes, int64_t page_bytes, int n_pages, const int* triples, int n,
                         cudaStream_t stream) {
    if (n <= 0 || planes <= 0) return 0;
    if (page_bytes <= 0 || (page_bytes & 15) || ((uintptr_t)base & 15) || (plane_stride & 15))
        GB_REFUSE("zero_pages: pages of %lld bytes, plane stride %lld: both must be multiples of 16", (long long)page_bytes, (long long)plane_stride);
    if (planes > 65535) GB_REFUSE("zero_pages: %d planes exceed one launch", planes);
    zero_pages_kernel<<<dim3(n, planes), 256, 0, stream>>>((unsigned char*)base, plane_stride, page_bytes, n_pages, triples);
    GB_CHECK_LAUNCH("zero_pages");
    return 0;
}

// ------------------------------------------------------------------------------------------
// Seeded fill.  Element i of a tensor with key `key` (a 64-bit digest of seed and tensor name, made
// on the host) is
//     s = sum of the eight 16-bit fields of word(2 i) and word(2 i + 1),
//     word(j) = splitmix64 finaliser of key + (j + 1) * 0x9E3779B97F4A7C15   (mod 2^64),
//     value   = fl32(fl32(s - 262140) * c) + mean,      c = fl32(std / sqrt(2 (2^32 - 1) / 3)),
// the sum of eight uniform 16-bit integers centred and scaled to the wanted deviation: integers up
// to 2^19 are exact in fp32, and one multiplication and one addition, each rounded once, give the
// same bits wherever they are computed, which a logarithm or a cosine would not.  The host
// writer of model folders computes the same function in numpy.
__device__ __forceinline__ unsigned long long fill_word(unsigned long long key, unsigned long long j) {
    unsigned long long x = key + (j + 1ull) * 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

__device__ __forceinline__ int fields16(unsigned long long w) {
    return (int)(w & 0xffffull) + (int)((w >> 16) & 0xffffull) + (int)((w >> 32) & 0xffffull) + (int)(w >> 48);
}

template <typename T>
__global__ void random_fill_kernel(T* __restrict__ out, int64_t n, unsigned long long key, float c, float mean) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const int s = fields16(fill_word(key, 2ull * (unsigned long long)i)) + fields16(fill_word(key, 2ull * (unsigned long long)i + 1ull));
        const float v = __fadd_rn(__fmul_rn((float)(s - 262140), c), mean);
        out[i] = from_f32<T>(v);
    }
}

GB_API int gb_random_fill(void* out, int dtype, int64_t n, unsigned long long key, float c, float mean, cudaStream_t stream) {
    if (n <= 0) return 0;
    int64_t blocks = (n + 1023) / 1024;
    if (blocks > 148 * 32) blocks = 148 * 32;
    if (dtype == GB_F32)
        random_fill_kernel<float><<<(unsigned)blocks, 256, 0, stream>>>((float*)out, n, key, c, mean);
    else if (dtype == GB_BF16)
        random_fill_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, stream>>>((__nv_bfloat16*)out, n, key, c, mean);
    else
        GB_REFUSE("random_fill: unknown dtype %d", dtype);
    GB_CHECK_LAUNCH("random_fill");
    return 0;
}

// the checked build's record of the first index this file's kernels found out of bounds
GB_CHECK_READER(gb_checked_status_cache)
