// Load-time repack: GGUF file blocks -> the planar device layout described at DevMatrix.
//
// The reference repacks on the CPU at load for its NEON kernels (src/model.cpp:481-525,
// src/quant.cpp:322-340, :616-633, :862-882, :927-951); here the raw file bytes are uploaded once and
// a kernel scatters them into 16-byte units plus scale planes, so a 4 GB model repacks in milliseconds.
// The repack is lossless: tests read the planes back and decode them bit-identically to the file blocks.
#include "kernels.h"

namespace bk {

static size_t align256(size_t v) { return (v + 255) & ~size_t(255); }

PlaneSizes plane_sizes(int type, uint32_t rows, uint32_t cols) {
    PlaneSizes p;
    const size_t r = rows;
    switch (type) {
        case T_F32: p.qa = r * cols * 4; break;
        case T_F16: p.qa = r * cols * 2; break;
        case T_Q4_0: p.qa = r * (cols / 32) * 16; p.d = r * (cols / 32) * 2; break;
        case T_Q4_1: p.qa = r * (cols / 32) * 16; p.d = r * (cols / 32) * 4; break;
        case T_Q5_0: p.qa = r * (cols / 32) * 16; p.qb = r * (cols / 32) * 4; p.d = r * (cols / 32) * 2; break;
        case T_Q8_0: p.qa = r * (cols / 32) * 32; p.d = r * (cols / 32) * 2; break;
        case T_Q5_K: p.qa = r * (cols / 256) * 128; p.qb = r * (cols / 256) * 32; p.sc = r * (cols / 256) * 16; p.d = r * (cols / 256) * 4; break;
        case T_Q4_K: p.qa = r * (cols / 256) * 128; p.sc = r * (cols / 256) * 16; p.d = r * (cols / 256) * 4; break;
        case T_Q6_K:
            p.qa = p.qb = p.qc = r * (cols / 256) * 64;
            p.sc = r * (cols / 256) * 16;
            p.d = r * (cols / 256) * 2;
            break;
        case T_TQ2_0: p.qa = r * (cols / 256) * 64; p.d = r * (cols / 256) * 2; break;
        default: break;
    }
    p.qa = align256(p.qa); p.qb = align256(p.qb); p.qc = align256(p.qc); p.sc = align256(p.sc); p.d = align256(p.d);
    return p;
}

void bind_planes(DevMatrix& m, int type, uint32_t rows, uint32_t cols, uint8_t* base) {
    const PlaneSizes p = plane_sizes(type, rows, cols);
    m.type = type;
    m.rows = rows;
    m.cols = cols;
    m.bytes = p.total();
    switch (type) {
        case T_Q4_0: case T_Q4_1: case T_Q5_0: m.units = cols / 32; m.blocks = cols / 32; break;
        case T_Q8_0: m.units = cols / 16; m.blocks = cols / 32; break;
        case T_Q4_K: case T_Q5_K: m.units = cols / 32; m.blocks = cols / 256; break;
        case T_Q6_K: m.units = cols / 64; m.blocks = cols / 256; break;
        case T_TQ2_0: m.units = cols / 64; m.blocks = cols / 256; break;
        case T_F16: m.units = cols / 8; m.blocks = 0; break;
        default: m.units = cols / 4; m.blocks = 0; break;
    }
    uint8_t* at = base;
    m.qa = at; at += p.qa;
    m.qb = p.qb ? at : nullptr; at += p.qb;
    m.qc = p.qc ? at : nullptr; at += p.qc;
    m.sc = p.sc ? at : nullptr; at += p.sc;
    m.d = p.d ? reinterpret_cast<const __half*>(at) : nullptr;
}

namespace {

__device__ __forceinline__ void copy16(uint8_t* dst, const uint8_t* src) {
    // File blocks are only 2-byte aligned, so gather bytes; the destination unit is 16-byte aligned.
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        w[i] = uint32_t(src[4 * i]) | (uint32_t(src[4 * i + 1]) << 8) | (uint32_t(src[4 * i + 2]) << 16) | (uint32_t(src[4 * i + 3]) << 24);
    }
    *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
}

__device__ __forceinline__ uint16_t load_u16(const uint8_t* p) { return uint16_t(p[0]) | (uint16_t(p[1]) << 8); }

__global__ void repack_kernel(int type, size_t total_units, const uint8_t* __restrict__ raw, uint8_t* qa, uint8_t* qb, uint8_t* qc,
                              uint8_t* sc, uint16_t* d) {
    const size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= total_units) return;
    switch (type) {
        case T_Q4_0: {
            const uint8_t* b = raw + i * 18;
            d[i] = load_u16(b);
            copy16(qa + i * 16, b + 2);
            break;
        }
        case T_Q4_1: {
            const uint8_t* b = raw + i * 20;
            d[2 * i] = load_u16(b);
            d[2 * i + 1] = load_u16(b + 2);
            copy16(qa + i * 16, b + 4);
            break;
        }
        case T_Q5_0: {
            const uint8_t* b = raw + i * 22;
            d[i] = load_u16(b);
            reinterpret_cast<uint32_t*>(qb)[i] = uint32_t(b[2]) | (uint32_t(b[3]) << 8) | (uint32_t(b[4]) << 16) | (uint32_t(b[5]) << 24);
            copy16(qa + i * 16, b + 6);
            break;
        }
        case T_Q8_0: {
            const size_t blk = i >> 1, half = i & 1;
            const uint8_t* b = raw + blk * 34;
            if (half == 0) d[blk] = load_u16(b);
            copy16(qa + i * 16, b + 2 + half * 16);
            break;
        }
        case T_Q4_K: {
            const size_t blk = i >> 3, j = i & 7;
            const uint8_t* b = raw + blk * 144;
            copy16(qa + i * 16, b + 16 + j * 16);
            if (j == 0) {
                d[2 * blk] = load_u16(b);
                d[2 * blk + 1] = load_u16(b + 2);
                const uint8_t* s = b + 4;  // 12 bytes of packed 6-bit scales and mins (src/quant.h:256-264)
                uint8_t* o = sc + blk * 16;
                for (int k = 0; k < 4; ++k) {
                    o[k] = s[k] & 63;
                    o[8 + k] = s[k + 4] & 63;
                    o[4 + k] = uint8_t((s[k + 8] & 0xF) | ((s[k] >> 6) << 4));
                    o[12 + k] = uint8_t((s[k + 8] >> 4) | ((s[k + 4] >> 6) << 4));
                }
            }
            break;
        }
        case T_Q5_K: {
            const size_t blk = i >> 3, j = i & 7, g = j >> 1, hf = j & 1;
            const uint8_t* b = raw + blk * 176;
            copy16(qa + i * 16, b + 48 + j * 16);
            const uint8_t* qh = b + 16 + hf * 16;  // bit sb of qh[e] is the fifth bit of value e of sub-block sb (src/quant.h:101-110)
            uint32_t bits = 0;
            for (int k = 0; k < 16; ++k) {
                bits |= uint32_t((qh[k] >> (2 * g)) & 1) << k;
                bits |= uint32_t((qh[k] >> (2 * g + 1)) & 1) << (16 + k);
            }
            reinterpret_cast<uint32_t*>(qb)[i] = bits;
            if (j == 0) {
                d[2 * blk] = load_u16(b);
                d[2 * blk + 1] = load_u16(b + 2);
                const uint8_t* s = b + 4;
                uint8_t* o = sc + blk * 16;
                for (int k = 0; k < 4; ++k) {
                    o[k] = s[k] & 63;
                    o[8 + k] = s[k + 4] & 63;
                    o[4 + k] = uint8_t((s[k + 8] & 0xF) | ((s[k] >> 6) << 4));
                    o[12 + k] = uint8_t((s[k + 8] >> 4) | ((s[k + 4] >> 6) << 4));
                }
            }
            break;
        }
        case T_Q6_K: {
            const size_t blk = i >> 2, c = i & 3, half = c >> 1, lr = (c & 1) * 16;
            const uint8_t* b = raw + blk * 210;
            copy16(qa + i * 16, b + half * 64 + lr);
            copy16(qb + i * 16, b + half * 64 + 32 + lr);
            copy16(qc + i * 16, b + 128 + half * 32 + lr);
            if (c == 0) {
                copy16(sc + blk * 16, b + 192);
                d[blk] = load_u16(b + 208);
            }
            break;
        }
        case T_TQ2_0: {
            const size_t blk = i >> 2, c = i & 3;
            const uint8_t* b = raw + blk * 66;
            copy16(qa + i * 16, b + c * 16);
            if (c == 0) d[blk] = load_u16(b + 64);
            break;
        }
        default: break;
    }
}

__global__ void widen_bf16_kernel(size_t count, const uint16_t* __restrict__ raw, float* out) {
    const size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < count) out[i] = __uint_as_float(uint32_t(raw[i]) << 16);  // bfloat_to_float, src/model.cpp:20-25
}

}  // namespace

void launch_widen_bf16(const DevMatrix& m, const uint8_t* raw_dev, cudaStream_t s) {
    const size_t count = size_t(m.rows) * m.cols;
    widen_bf16_kernel<<<unsigned((count + 255) / 256), 256, 0, s>>>(count, reinterpret_cast<const uint16_t*>(raw_dev),
                                                                    reinterpret_cast<float*>(const_cast<uint8_t*>(m.qa)));
    BK_CUDA(cudaGetLastError());
}

void launch_repack(const DevMatrix& m, const uint8_t* raw_dev, cudaStream_t s) {
    if (m.type == T_F32 || m.type == T_F16) {
        BK_CUDA(cudaMemcpyAsync(const_cast<uint8_t*>(m.qa), raw_dev, size_t(m.rows) * m.cols * (m.type == T_F32 ? 4 : 2),
                                cudaMemcpyDeviceToDevice, s));
        return;
    }
    const size_t total = size_t(m.rows) * m.units;
    const unsigned threads = 256;
    const unsigned grid = unsigned((total + threads - 1) / threads);
    repack_kernel<<<grid, threads, 0, s>>>(m.type, total, raw_dev, const_cast<uint8_t*>(m.qa), const_cast<uint8_t*>(m.qb),
                                           const_cast<uint8_t*>(m.qc), const_cast<uint8_t*>(m.sc),
                                           reinterpret_cast<uint16_t*>(const_cast<__half*>(m.d)));
    BK_CUDA(cudaGetLastError());
}

}  // namespace bk
