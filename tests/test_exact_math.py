"""exact_math.h on the host: the restated single-precision exp must equal the C library's expf bit for bit - it exists
so that SiLU and softmax on the GPU produce the floats the reference CPU engine (which calls libm) produces."""
import os
import subprocess
import tempfile
import textwrap

import helpers as H

SRC = textwrap.dedent(r'''
    #include <cmath>
    #include <cstdint>
    #include <cstdio>
    #include <cstring>
    #include "exact_math.h"
    int main() {
        uint64_t bad = 0, n = 0;
        uint32_t st = 2463534242u;
        for (uint64_t it = 0; it < 30000000ull; ++it) {
            st = st * 1664525u + 1013904223u;
            float x;
            std::memcpy(&x, &st, 4);
            if (!(x == x)) continue;
            if (std::fabs(x) > 110.0f) x = std::fmod(x, 110.0f);
            const float a = bk::exact_expf(x), b = std::exp(x);
            n++;
            if (std::memcmp(&a, &b, 4) != 0) bad++;
        }
        // the ranges the token loop uses densely: softmax arguments (<= 0) and SiLU arguments around 0
        for (float x = -12.0f; x < 4.0f; x += 1.9073486e-06f) {
            const float a = bk::exact_expf(x), b = std::exp(x);
            n++;
            if (std::memcmp(&a, &b, 4) != 0) bad++;
        }
        const float edge[] = {0.0f, -0.0f, 88.7f, 88.73f, 89.0f, -87.0f, -88.0f, -95.0f, -103.9f, -104.0f, -1e30f, 1e30f};
        for (float x : edge) {
            const float a = bk::exact_expf(x), b = std::exp(x);
            n++;
            if (std::memcmp(&a, &b, 4) != 0) bad++;
        }
        std::printf("%llu %llu\n", (unsigned long long)n, (unsigned long long)bad);
        return 0;
    }''')


def test_exact_expf_matches_the_host_libm():
    with tempfile.TemporaryDirectory() as d:
        src, exe = os.path.join(d, "t.cpp"), os.path.join(d, "t")
        open(src, "w").write(SRC)
        subprocess.run(["g++", "-O2", "-ffp-contract=off", "-I", os.path.join(H.ROOT, "brisk_llm_b200", "csrc"), src, "-o", exe], check=True)
        n, bad = (int(v) for v in subprocess.run([exe], capture_output=True, text=True, check=True).stdout.split())
    assert n > 30_000_000 and bad == 0, (n, bad)
