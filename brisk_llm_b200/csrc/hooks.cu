// Standalone multiply entry points of the C ABI: the test hook and the bench hook, counterparts of the
// Metal backend's metal_matmul / metal_matmul_seconds (src/metal/metal_session.h:39-59).
#include <cstdio>
#include <string>
#include <vector>

#include "../../include/brisk_cuda.h"
#include "kernels.h"

namespace {

struct Buf {
    void* p = nullptr;
    explicit Buf(size_t n) { BK_CUDA(cudaMalloc(&p, n ? n : 16)); }
    Buf(const Buf&) = delete;
    ~Buf() { cudaFree(p); }
    template <class T> T* as() const { return static_cast<T*>(p); }
};

void put_error(char* err, size_t errlen, const std::string& what) {
    if (err != nullptr && errlen > 0) std::snprintf(err, errlen, "%s", what.c_str());
}

void validate(int32_t type, uint64_t rows, uint64_t cols) {
    const uint32_t be = bk::block_elems(type);
    if (bk::block_bytes(type) == 0) throw bk::CudaError("cuda: unsupported weight type " + std::to_string(type));
    if (rows == 0 || cols == 0 || cols % be != 0 || cols % 32 != 0) throw bk::CudaError("cuda: row length is not a multiple of the block size");
}

struct ActBuffers {
    Buf f32, q0, d0, s0, qk, dk, bs;
    bk::DevActMut act;
    ActBuffers(uint64_t n, uint64_t cols)
        : f32(n * cols * 4), q0(n * cols), d0(n * (cols / 32) * 4), s0(n * (cols / 32) * 4), qk(n * cols), dk(n * (cols / 256 + 1) * 4),
          bs(n * (cols / 16) * 2) {
        act.f32 = f32.as<float>(); act.q0 = q0.as<int8_t>(); act.d0 = d0.as<float>(); act.s0 = s0.as<int32_t>();
        act.qk = qk.as<int8_t>(); act.dk = dk.as<float>(); act.bs = bs.as<int16_t>(); act.cols = uint32_t(cols);
    }
};

// The multiply the session would run for n tokens: the fused single-token kernel (which quantises x itself), the
// few-token kernel or the streaming kernel for small batches, the tensor-core kernel for prompt batches.
void multiply(const bk::DevMatrix& m, float* out, const float* x, const bk::DevAct& a, uint32_t n, uint32_t sms, cudaStream_t s) {
    bk::MatTarget t{m, out, m.rows};
    if (n == 1) {
        bk::launch_dec_multiply(&t, 1, x, nullptr, 0.0f, m.cols, bk::EPI_STORE, sms, s);
    } else if (bk::launch_smallbatch(&t, 1, a, n, bk::EPI_STORE, s)) {
        // 2..16 tokens of a Q4_0 / Q8_0 matrix
    } else if (!(n >= 16 && bk::launch_gemm(&t, 1, a, n, bk::EPI_STORE, s))) {
        bk::launch_matvec(&t, 1, a, n, bk::EPI_STORE, s);
    }
}

uint32_t sm_count() {
    int dev = 0, count = 0;
    BK_CUDA(cudaGetDevice(&dev));
    BK_CUDA(cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, dev));
    return uint32_t(count);
}

}  // namespace

extern "C" {

int brisk_cuda_matmul(int32_t type, const void* w, uint64_t rows, uint64_t cols, const float* x, uint64_t n, float* out, char* err,
                      size_t errlen) {
    try {
        if (brisk_cuda_device_count() < 1) throw bk::CudaError("cuda: no usable CUDA device (this backend has no CPU path)");
        validate(type, rows, cols);
        if (n == 0) return 0;
        const size_t raw_bytes = rows * (cols / bk::block_elems(type)) * bk::block_bytes(type);
        const int dev_type = type == bk::T_BF16 ? int(bk::T_F32) : type;  // BF16 is widened on upload
        Buf raw(raw_bytes), planes(bk::plane_sizes(dev_type, uint32_t(rows), uint32_t(cols)).total()), xd(n * cols * 4), od(n * rows * 4);
        ActBuffers ab(n, cols);
        bk::DevMatrix m;
        bk::bind_planes(m, dev_type, uint32_t(rows), uint32_t(cols), planes.as<uint8_t>());
        BK_CUDA(cudaMemcpy(raw.p, w, raw_bytes, cudaMemcpyHostToDevice));
        BK_CUDA(cudaMemcpy(xd.p, x, n * cols * 4, cudaMemcpyHostToDevice));
        if (type == bk::T_BF16) bk::launch_widen_bf16(m, raw.as<uint8_t>(), nullptr);
        else bk::launch_repack(m, raw.as<uint8_t>(), nullptr);
        const bool k = bk::takes_q8_k(type), f = type == bk::T_F16 || type == bk::T_F32 || type == bk::T_BF16;
        bk::DevActMut a = ab.act;
        if (!f) a.f32 = nullptr;
        bk::launch_norm_quant(xd.as<float>(), uint32_t(cols), nullptr, 0.0f, uint32_t(n), uint32_t(cols), a, !k && !f, k, nullptr);
        multiply(m, od.as<float>(), xd.as<float>(), ab.act.view(), uint32_t(n), sm_count(), nullptr);
        BK_CUDA(cudaMemcpy(out, od.p, n * rows * 4, cudaMemcpyDeviceToHost));
        return 0;
    } catch (const std::exception& e) {
        put_error(err, errlen, e.what());
        return -1;
    }
}

int brisk_cuda_matmul_seconds(int32_t type, const void* w, uint64_t rows, uint64_t cols, uint64_t n, uint32_t copies, uint32_t iterations,
                              double* seconds, char* err, size_t errlen) {
    try {
        if (brisk_cuda_device_count() < 1) throw bk::CudaError("cuda: no usable CUDA device (this backend has no CPU path)");
        validate(type, rows, cols);
        if (n == 0 || copies == 0 || iterations == 0) throw bk::CudaError("cuda: n, copies and iterations must be positive");
        const size_t raw_bytes = rows * (cols / bk::block_elems(type)) * bk::block_bytes(type);
        const size_t plane_bytes = bk::plane_sizes(type, uint32_t(rows), uint32_t(cols)).total();
        Buf raw(raw_bytes), planes(plane_bytes * copies), xd(n * cols * 4), od(n * rows * 4);
        ActBuffers ab(n, cols);
        BK_CUDA(cudaMemcpy(raw.p, w, raw_bytes, cudaMemcpyHostToDevice));
        std::vector<bk::DevMatrix> ms(copies);
        for (uint32_t c = 0; c < copies; ++c) {
            bk::bind_planes(ms[c], type, uint32_t(rows), uint32_t(cols), planes.as<uint8_t>() + size_t(c) * plane_bytes);
            bk::launch_repack(ms[c], raw.as<uint8_t>(), nullptr);
        }
        // Activations: a fixed pseudo-random f32 pattern (values do not change the timing).
        std::vector<float> xh(n * cols);
        uint32_t state = 12345u;
        for (float& v : xh) {
            state = state * 1664525u + 1013904223u;
            v = float(int32_t(state >> 8) % 2001 - 1000) / 1000.0f;
        }
        BK_CUDA(cudaMemcpy(xd.p, xh.data(), xh.size() * 4, cudaMemcpyHostToDevice));
        const bool k = bk::takes_q8_k(type), f = type == bk::T_F16 || type == bk::T_F32;
        bk::launch_norm_quant(xd.as<float>(), uint32_t(cols), nullptr, 0.0f, uint32_t(n), uint32_t(cols), ab.act, !k && !f, k, nullptr);
        const uint32_t sms = sm_count();
        for (uint32_t i = 0; i < 3; ++i) multiply(ms[i % copies], od.as<float>(), xd.as<float>(), ab.act.view(), uint32_t(n), sms, nullptr);
        cudaEvent_t e0, e1;
        BK_CUDA(cudaEventCreate(&e0));
        BK_CUDA(cudaEventCreate(&e1));
        BK_CUDA(cudaEventRecord(e0, nullptr));
        for (uint32_t i = 0; i < iterations; ++i) multiply(ms[i % copies], od.as<float>(), xd.as<float>(), ab.act.view(), uint32_t(n), sms, nullptr);
        BK_CUDA(cudaEventRecord(e1, nullptr));
        BK_CUDA(cudaEventSynchronize(e1));
        float ms_total = 0;
        BK_CUDA(cudaEventElapsedTime(&ms_total, e0, e1));
        cudaEventDestroy(e0);
        cudaEventDestroy(e1);
        *seconds = double(ms_total) * 1e-3 / iterations;
        return 0;
    } catch (const std::exception& e) {
        put_error(err, errlen, e.what());
        return -1;
    }
}

}  // extern "C"
