// The few extra kernels of the Gemma 3 layer variants (brisk-llm src/model.h:24): the embedding scale, the RMS norm a
// projection's output gets before it joins the residual stream, the soft cap of the logits, and the table that lets the
// device's tanh reproduce the host C library's tanhf. The tanh-GELU gate is gelu_mul() in formats.cuh, applied by
// launch_gate_mul; the sliding window is a parameter of the attention kernels.
#include <algorithm>
#include <cmath>
#include <cstring>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "common.cuh"
#include "formats.cuh"
#include "kernels.h"
#include "rowops.cuh"

namespace bk {
namespace {

__global__ void __launch_bounds__(256) scale_rows_kernel(float* x, size_t count, float scale) {
    const size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < count) x[i] = __fmul_rn(x[i], scale);
}

// One CTA per token row: p = proj * scale * weight (rms_norm's order, src/model.cpp:87-97), then hidden += p.
__global__ void __launch_bounds__(256) post_norm_add_kernel(const float* __restrict__ proj, const float* __restrict__ weight,
                                                            float* __restrict__ hidden, uint32_t cols, float eps) {
    __shared__ double red[32];
    const float* p = proj + size_t(blockIdx.x) * cols;
    float* h = hidden + size_t(blockIdx.x) * cols;
    const float scale = cta_rms_scale(p, cols, eps, red);
    for (uint32_t i = threadIdx.x; i < cols; i += blockDim.x) {
        h[i] = __fadd_rn(h[i], __fmul_rn(__fmul_rn(p[i], scale), weight[i]));
    }
}

__global__ void __launch_bounds__(256) softcap_kernel(float* logits, size_t count, float cap, const uint8_t* tanh_table) {
    const size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < count) logits[i] = __fmul_rn(cap, tanh_like_host(__fdiv_rn(logits[i], cap), tanh_table));
}

// out[i] = the device's base tanh of the float whose bits are first + i.
__global__ void __launch_bounds__(256) tanh_base_kernel(uint32_t first, uint32_t count, float* out) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < count) out[i] = tanh_base(__uint_as_float(first + i));
}

}  // namespace

void launch_scale_rows(float* x, size_t count, float scale, cudaStream_t s) {
    scale_rows_kernel<<<unsigned((count + 255) / 256), 256, 0, s>>>(x, count, scale);
    BK_CUDA(cudaGetLastError());
}

void launch_post_norm_add(const float* proj, const float* weight, float* hidden, uint32_t n, uint32_t cols, float eps, cudaStream_t s) {
    post_norm_add_kernel<<<n, 256, 0, s>>>(proj, weight, hidden, cols, eps);
    BK_CUDA(cudaGetLastError());
}

void launch_softcap(float* logits, size_t count, float cap, const uint8_t* tanh_table, cudaStream_t s) {
    softcap_kernel<<<unsigned((count + 255) / 256), 256, 0, s>>>(logits, count, cap, tanh_table);
    BK_CUDA(cudaGetLastError());
}

size_t tanh_table_bytes() { return size_t(kTanhTableHi - kTanhTableLo) / 2; }

void build_tanh_table(uint8_t* table, unsigned threads, cudaStream_t s) {
    constexpr uint32_t kChunk = 1u << 24;  // floats per round trip (64 MB of base values)
    const uint32_t total = kTanhTableHi - kTanhTableLo;
    threads = std::max(1u, std::min(threads, 64u));
    // Two device buffers and two pinned host buffers: the device evaluates and copies chunk i + 1 while the host threads
    // work on chunk i.
    struct Buffers {
        float* dev[2] = {nullptr, nullptr};
        float* host[2] = {nullptr, nullptr};
        ~Buffers() {
            for (int i = 0; i < 2; ++i) {
                if (dev[i]) cudaFree(dev[i]);
                if (host[i]) cudaFreeHost(host[i]);
            }
        }
    } buf;
    for (int i = 0; i < 2; ++i) {
        BK_CUDA(cudaMalloc(&buf.dev[i], size_t(kChunk) * sizeof(float)));
        BK_CUDA(cudaMallocHost(&buf.host[i], size_t(kChunk) * sizeof(float)));
    }
    std::vector<uint8_t> packed(tanh_table_bytes());
    std::string failure;
    std::mutex failure_lock;
    // Outside the table both sides must agree by themselves: tanhf(x) == x below 2^-25 and == 1 from 22 on (the device's
    // base function returns exactly that). Sampled, every 65537th float, so that a C library for which this does not hold
    // is refused instead of silently disagreeing.
    auto outside = [&](uint32_t first, uint32_t last, bool small) {
        for (uint32_t u = first; u < last; u += 65537u) {
            float x;
            std::memcpy(&x, &u, sizeof x);
            const float want = small ? x : 1.0f, got = ::tanhf(x);
            if (std::memcmp(&want, &got, sizeof want) != 0) {
                throw CudaError("cuda: the host library's tanhf leaves the range the correction table covers (set BRISK_CUDA_TANH_TABLE=0 to run without it)");
            }
        }
    };
    outside(1u, kTanhTableLo, true);
    outside(kTanhTableHi, 0x7f800000u, false);
    auto request = [&](uint32_t c0, int slot) {
        const uint32_t n = std::min(kChunk, total - c0);
        tanh_base_kernel<<<(n + 255) / 256, 256, 0, s>>>(kTanhTableLo + c0, n, buf.dev[slot]);
        BK_CUDA(cudaGetLastError());
        BK_CUDA(cudaMemcpyAsync(buf.host[slot], buf.dev[slot], size_t(n) * sizeof(float), cudaMemcpyDeviceToHost, s));
    };
    request(0, 0);
    int slot = 0;
    for (uint32_t c0 = 0; c0 < total; c0 += kChunk, slot ^= 1) {
        const uint32_t n = std::min(kChunk, total - c0);  // even: kChunk and total are
        BK_CUDA(cudaStreamSynchronize(s));                 // chunk c0 is in buf.host[slot]
        if (c0 + kChunk < total) request(c0 + kChunk, slot ^ 1);
        const float* base = buf.host[slot];
        auto work = [&, base, c0](uint32_t lo, uint32_t hi) {  // [lo, hi) of this chunk, lo and hi even
            for (uint32_t i = lo; i < hi; i += 2) {
                uint8_t byte = 0;
                for (uint32_t k = 0; k < 2; ++k) {
                    const uint32_t in = kTanhTableLo + c0 + i + k;
                    float x;
                    std::memcpy(&x, &in, sizeof x);
                    const float want = ::tanhf(x);  // the C library's tanhf: what std::tanh on a float calls in the CPU engine
                    int32_t wb, bb;
                    std::memcpy(&wb, &want, sizeof wb);
                    std::memcpy(&bb, &base[i + k], sizeof bb);
                    const int64_t delta = int64_t(wb) - int64_t(bb);
                    if (delta < -8 || delta > 7) {
                        std::lock_guard<std::mutex> g(failure_lock);
                        failure = "cuda: the host library's tanhf and the device's differ by more than 8 units in the last place";
                        return;
                    }
                    byte |= uint8_t(delta + 8) << (4 * k);
                }
                packed[(size_t(c0) + i) / 2] = byte;
            }
        };
        std::vector<std::thread> pool;
        const uint32_t per = ((n / 2 + threads - 1) / threads) * 2;
        for (uint32_t t = 0; t < threads; ++t) {
            const uint32_t lo = std::min(n, t * per), hi = std::min(n, lo + per);
            if (lo < hi) pool.emplace_back(work, lo, hi);
        }
        for (std::thread& t : pool) t.join();
        if (!failure.empty()) break;
    }
    BK_CUDA(cudaStreamSynchronize(s));
    if (!failure.empty()) throw CudaError(failure);
    BK_CUDA(cudaMemcpyAsync(table, packed.data(), packed.size(), cudaMemcpyHostToDevice, s));
    BK_CUDA(cudaStreamSynchronize(s));
}

}  // namespace bk
