"""The allocation-free arg-max entry point (brisk_cuda_argmax_static), called through the C ABI.

It exists for hosts that cannot allocate device memory when they need a greedy pick: a server that has given all of
HBM to its own K/V arena, or a latency-critical thread that must not hit the device-wide synchronisation an allocation
implies. Its reduction scratch is a fixed array inside the library instead of a cudaMalloc'd buffer. The check: it
must pick exactly the tokens the existing greedy entry point (brisk_cuda_generate_greedy, whose arg-max uses allocated
scratch) picked from the same logits - on two calls in a row, so a call cannot depend on what the previous one left
in the shared scratch. This file sorts last on purpose.
"""
import ctypes as C

import numpy as np
import pytest

import helpers as H  # noqa: F401  (puts the repository on sys.path)
from brisk_llm_b200 import abi, engine, synth

pytestmark = pytest.mark.gpu


def static_argmax(lib, logits_dev, out_dev, rows, vocab, stream):
    err = C.create_string_buffer(256)
    rc = lib.brisk_cuda_argmax_static(logits_dev.data_ptr(), vocab, rows, out_dev.data_ptr(), stream, err, len(err))
    return rc, err.value.decode()


def test_static_argmax_matches_the_greedy_entry_point_twice_in_a_row():
    import torch
    lib = abi.load_library()
    spec = synth.tiny(synth.QWEN3_0_6B, layers=2, vocab=4096, context=128)
    model = synth.generate(spec, seed=4)
    prompt = synth.random_tokens(spec, 12, seed=5)
    with engine.CudaSession(model) as s:
        s.eval(prompt[:11])
        ids, logits = s.generate_greedy(int(prompt[11]), 9, want_logits=True)  # the existing entry point's picks
    assert list(ids) == [int(np.argmax(row)) for row in logits]  # first maximum, as the host sampler picks

    dev = torch.device("cuda", 0)
    stream = torch.cuda.current_stream(dev).cuda_stream
    first = torch.from_numpy(logits).to(dev)
    out = torch.full((9,), -1, dtype=torch.int32, device=dev)
    rc, msg = static_argmax(lib, first, out, 9, spec.vocab, stream)
    assert rc == 0, msg
    torch.cuda.synchronize()
    assert out.cpu().tolist() == list(ids)

    # second call straight after, other rows in another order and fewer of them: nothing may leak from the first call
    order = [7, 2, 5]
    second = torch.from_numpy(np.ascontiguousarray(logits[order])).to(dev)
    out2 = torch.full((3,), -1, dtype=torch.int32, device=dev)
    rc, msg = static_argmax(lib, second, out2, 3, spec.vocab, stream)
    assert rc == 0, msg
    torch.cuda.synchronize()
    assert out2.cpu().tolist() == [int(ids[i]) for i in order]


def test_static_argmax_ties_and_limits():
    import torch
    lib = abi.load_library()
    dev = torch.device("cuda", 0)
    stream = torch.cuda.current_stream(dev).cuda_stream
    rows = torch.zeros((2, 1000), dtype=torch.float32, device=dev)
    rows[1, 400] = 3.0
    rows[1, 900] = 3.0  # equal maxima: the lower id wins
    out = torch.full((2,), -1, dtype=torch.int32, device=dev)
    rc, msg = static_argmax(lib, rows, out, 2, 1000, stream)
    assert rc == 0, msg
    torch.cuda.synchronize()
    assert out.cpu().tolist() == [0, 400]
    too_many = torch.zeros((65, 8), dtype=torch.float32, device=dev)
    out65 = torch.zeros((65,), dtype=torch.int32, device=dev)
    rc, msg = static_argmax(lib, too_many, out65, 65, 8, stream)
    assert rc != 0 and "at most 64 rows" in msg


def test_static_argmax_follows_max_element_on_nan():
    """std::max_element (brisk-llm src/sampler.cpp:11-13) never prefers a NaN and never leaves one that sits at index 0:
    the pick stays inside the vocabulary whatever the row holds. The call only reads the caller's buffer."""
    import torch
    lib = abi.load_library()
    dev = torch.device("cuda", 0)
    stream = torch.cuda.current_stream(dev).cuda_stream
    nan = float("nan")
    rows = torch.zeros((5, 3000), dtype=torch.float32, device=dev)
    rows[0, :] = nan                      # nothing but NaN: the first element stays
    rows[1, 100] = nan                    # NaN among numbers is skipped ...
    rows[1, 2500] = 2.0                   # ... the first maximum of the rest wins
    rows[1, 2900] = 2.0
    rows[2, 0] = nan                      # a NaN in front is never displaced
    rows[2, 7] = 9.0
    rows[3, :] = -float("inf")            # equal values: the first
    rows[4, :] = -float("inf")
    rows[4, 1234] = nan
    rows[4, 2000] = -1.0
    out = torch.full((5,), -1, dtype=torch.int32, device=dev)
    rc, msg = static_argmax(lib, rows, out, 5, 3000, stream)
    assert rc == 0, msg
    torch.cuda.synchronize()
    host = rows.cpu().numpy()
    want = []
    for r in host:  # the loop of std::max_element
        best = 0
        for i in range(1, len(r)):
            if r[best] < r[i]:
                best = i
        want.append(best)
    assert want == [0, 2500, 0, 0, 2000]
    assert out.cpu().tolist() == want
