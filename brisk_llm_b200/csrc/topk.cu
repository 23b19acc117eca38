// The k best (id, logit) pairs of one logits row, on the device: what a sampling host needs instead of the whole row.
//
// The reference sampler (src/sampler.cpp:15-46) orders all candidates by value with std::partial_sort, keeps top_k of them,
// and runs its softmax, top-p cut and draw on those alone. Everything after the partial sort needs only the k pairs, so a
// backend that returns them (k * 8 bytes) spares the host the vocabulary-sized row (608 KB for 151 936 ids) per token.
//
// Selection is a small tree of bitonic sorts in shared memory. Level 0: every CTA sorts 1024 logits of the row as 64-bit
// keys - the value mapped so that larger sorts first, then the id, so equal values keep the lower id in front - and keeps
// its first k. Each further level sorts up to 1024 surviving keys per CTA and keeps k, until one CTA is left: three
// launches for vocabularies up to 16 M / k ids. A NaN sorts last (std::max_element and partial_sort never prefer one).
#include "kernels.h"

namespace bk {
namespace {

constexpr uint32_t kSortN = 1024;
constexpr uint32_t kSortThreads = 512;
constexpr unsigned long long kWorstKey = ~0ull;

__device__ __forceinline__ unsigned long long key_of(float v, uint32_t id) {
    uint32_t u = __float_as_uint(v);
    u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);  // ascending with the value
    if (v != v) u = 0;                                // NaN: below everything
    return (static_cast<unsigned long long>(~u) << 32) | id;  // ascending key = descending value, then ascending id
}
__device__ __forceinline__ float value_of(unsigned long long key) {
    uint32_t u = ~uint32_t(key >> 32);
    u = (u & 0x80000000u) ? (u & 0x7fffffffu) : ~u;
    return __uint_as_float(u);
}

// Sorts its up-to-1024 inputs, writes the first k keys to keys_out[cta][k]. level0: inputs are logits[cta * 1024 ..) of
// `count` values; else keys_in holds lists of k keys and this CTA takes `lists_per_cta` of the `count` lists.
__global__ void __launch_bounds__(kSortThreads) topk_level_kernel(const float* logits, const unsigned long long* keys_in, uint32_t count, uint32_t k,
                                                                  uint32_t lists_per_cta, unsigned long long* keys_out, int32_t* out_ids, float* out_values) {
    __shared__ unsigned long long keys[kSortN];
    const uint32_t tid = threadIdx.x, cta = blockIdx.x;
    for (uint32_t i = tid; i < kSortN; i += kSortThreads) {
        unsigned long long key = kWorstKey;
        if (logits != nullptr) {
            const uint32_t id = cta * kSortN + i;
            if (id < count) key = key_of(logits[id], id);
        } else {
            const uint32_t list = cta * lists_per_cta + i / k;
            if (i < lists_per_cta * k && list < count) key = keys_in[size_t(list) * k + i % k];
        }
        keys[i] = key;
    }
    __syncthreads();
    for (uint32_t size = 2; size <= kSortN; size <<= 1) {
        for (uint32_t stride = size >> 1; stride > 0; stride >>= 1) {
            for (uint32_t t = tid; t < kSortN / 2; t += kSortThreads) {
                const uint32_t lo = 2 * t - (t & (stride - 1)), hi = lo + stride;
                const bool up = (lo & size) == 0;
                const unsigned long long a = keys[lo], b = keys[hi];
                if ((a > b) == up) {
                    keys[lo] = b;
                    keys[hi] = a;
                }
            }
            __syncthreads();
        }
    }
    if (tid < k) {
        if (out_ids != nullptr) {  // the last level: the answer itself
            const unsigned long long key = keys[tid];
            out_ids[tid] = key == kWorstKey ? -1 : int32_t(uint32_t(key));
            out_values[tid] = key == kWorstKey ? -INFINITY : value_of(key);
        } else {
            keys_out[size_t(cta) * k + tid] = keys[tid];
        }
    }
}

}  // namespace

size_t topk_scratch_keys(uint32_t vocab, uint32_t k) {
    const size_t level0 = (size_t(vocab) + kSortN - 1) / kSortN;
    return 2 * level0 * k;  // two buffers: a level reads one and writes the other
}

void launch_topk(const float* logits, uint32_t vocab, uint32_t k, unsigned long long* scratch, int32_t* out_ids, float* out_values, cudaStream_t s,
                 uint64_t* launches) {
    if (k == 0 || k > kMaxTopK) throw CudaError("cuda: top-k takes k from 1 to " + std::to_string(kMaxTopK));
    uint32_t lists = (vocab + kSortN - 1) / kSortN;
    unsigned long long* a = scratch;
    unsigned long long* b = scratch + size_t(lists) * k;
    const bool single = lists == 1;
    topk_level_kernel<<<lists, kSortThreads, 0, s>>>(logits, nullptr, vocab, k, 0, a, single ? out_ids : nullptr, single ? out_values : nullptr);
    BK_CUDA(cudaGetLastError());
    if (launches) ++*launches;
    const uint32_t per_cta = kSortN / k;
    while (lists > 1) {
        const uint32_t ctas = (lists + per_cta - 1) / per_cta;
        const bool last = ctas == 1;
        topk_level_kernel<<<ctas, kSortThreads, 0, s>>>(nullptr, a, lists, k, per_cta, b, last ? out_ids : nullptr, last ? out_values : nullptr);
        BK_CUDA(cudaGetLastError());
        if (launches) ++*launches;
        std::swap(a, b);
        lists = ctas;
    }
}

}  // namespace bk
