"""CPU checks of the drop-in boundary: the shared library loads without a GPU, exports every
symbol declared in include/jasmine_b200.h, validates arguments on the host with the
reference's error classes, and generates the same seeded data as the oracle."""
import ctypes as C
import re
from pathlib import Path

import numpy as np
import pytest

import jasmine_b200 as jb
import oracle_lib as ol

ROOT = Path(__file__).resolve().parents[1]


def declared_symbols():
    text = (ROOT / "include" / "jasmine_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(jsm_[a-z0-9_]+)\s*\(", text)) - {"jsm_allreduce_fn"})


def test_library_loads_and_exports_every_declared_symbol():
    L = jb.lib()
    names = declared_symbols()
    assert len(names) >= 30
    for n in names:
        assert hasattr(L, n), f"{n} is declared in the header but not exported"
        assert n in jb.SYMBOLS, f"{n} has no ctypes signature in jasmine_b200.SYMBOLS"
    assert L.jsm_version() >= 100


def test_fill_host_matches_oracle_generator():
    import torch
    for dist, a, b in ((0, 0.0, 0.02), (0, 1.0, 3.0), (1, 0.5, 1.5)):
        t = torch.empty(4097, dtype=torch.float32)
        jb.fill(t, 11, 5, dist, a, b)
        assert np.array_equal(t.numpy(), ol.fill(4097, 11, 5, dist, a, b))
    t = torch.empty(513, dtype=torch.int32)
    jb.fill(t, 3, 9, 2, 0, 32000)
    assert np.array_equal(t.numpy(), ol.fill(513, 3, 9, 2, 0, 32000).astype(np.int32))
    tb = torch.empty(1000, dtype=torch.bfloat16)
    jb.fill(tb, 4, 1, 0, 0.0, 0.02)
    assert np.array_equal(tb.float().numpy(), ol.fill(1000, 4, 1, 0, 0.0, 0.02, to_bf16=True))


def _mat(rows, cols, ptr=1 << 20):
    return jb.Mat(ptr, rows, cols, cols, 1, jb.F32)


def test_dot_shape_mismatch_is_invalid_argument():
    # mat_dot_t throws std::invalid_argument (mat_express_t.hpp:709-712); checked before any device work
    L = jb.lib()
    st = L.jsm_dot_f32(_mat(3, 4), _mat(5, 2), None, 0, None, _mat(3, 2), None)
    assert st == jb.INVALID_ARG
    assert b"inner dimensions do not match" in L.jsm_last_error()


def test_program_validation_on_host():
    L = jb.lib()
    leaves = (jb.Mat * 1)(_mat(4, 8))
    bad, n = jb.program([(jb.OP_LEAF, 0), (jb.OP_ADD,)])  # stack underflow
    assert L.jsm_eval_elementwise(bad, n, leaves, 1, _mat(4, 8), None) == jb.INVALID_ARG
    two, n = jb.program([(jb.OP_LEAF, 0), (jb.OP_LEAF, 0)])  # two values left
    assert L.jsm_eval_elementwise(two, n, leaves, 1, _mat(4, 8), None) == jb.INVALID_ARG
    ok, n = jb.program([(jb.OP_LEAF, 0), (jb.OP_EXP,)])
    assert L.jsm_eval_elementwise(ok, n, leaves, 1, _mat(4, 9), None) == jb.SHAPE  # result is 4 x 8
    assert L.jsm_eval_rows(99, 1, ok, n, leaves, 1, None, None, 0.0, _mat(4, 8), None) == jb.INVALID_ARG


def test_model_config_validation_on_host():
    L = jb.lib()
    h = C.c_void_p()
    cfg = jb.ModelConfig(2, 256, 3, 2, 128, 512, 1000, 1, 128, 1e-5, 10000.0, 0, 1)  # 3 heads over 2 kv heads
    assert L.jsm_llama_create(C.byref(cfg), 0, C.byref(h)) == jb.SHAPE
    cfg = jb.ModelConfig(2, 256, 2, 2, 64, 512, 1000, 1, 128, 1e-5, 10000.0, 0, 1)  # head_dim 64
    assert L.jsm_llama_create(C.byref(cfg), 0, C.byref(h)) == jb.UNSUPPORTED


def test_no_cpu_fallback_without_a_device():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    L = jb.lib()
    n = C.c_int(-1)
    assert L.jsm_device_count(C.byref(n)) == jb.CUDA and n.value == 0
    h = C.c_void_p()
    cfg = jb.ModelConfig(1, 256, 2, 2, 128, 512, 1000, 1, 128, 1e-5, 10000.0, 0, 1)
    assert L.jsm_llama_create(C.byref(cfg), 0, C.byref(h)) == jb.CUDA
    p = C.c_void_p()
    assert L.jsm_malloc(C.byref(p), 1024) in (jb.CUDA, jb.OOM)


@pytest.mark.parametrize("N,K,paired", [(4096, 4096, 0), (12288, 4096, 0), (11008, 4096, 1), (4096, 11008, 0), (32000, 4096, 0),
                                        (1376, 4096, 1), (4096, 1376, 0), (256, 512, 0), (1000, 1000, 0), (384, 64, 0),
                                        (704, 1024, 1), (4096, 512, 0)])
def test_packed_projection_work_split_is_consistent(N, K, paired):
    """The stream-K split of a packed projection, checked on the host: the CTA ranges tile the unit space, the owner
    formula inverts the range formula (it decides which workspace slot a CTA writes), and no tile has more
    contributors than the workspace has slots."""
    nt, kbt, G, slots = C.c_int(), C.c_int(), C.c_int(), C.c_int()
    assert jb.lib().jsm_linear_packed_plan(N, K, paired, C.byref(nt), C.byref(kbt), C.byref(G), C.byref(slots)) == jb.OK
    nt, kbt, G, slots = nt.value, kbt.value, G.value, slots.value
    assert nt == (-(-N // 64) if paired else -(-N // 128)) and kbt == -(-K // 64)
    U = nt * kbt
    assert 1 <= G <= 148 or G == U // 4
    begin = [c * U // G for c in range(G + 1)]
    assert begin[0] == 0 and begin[G] == U and all(b1 > b0 for b0, b1 in zip(begin, begin[1:]))
    owner = lambda u: ((u + 1) * G + U - 1) // U - 1
    for c in range(G):
        assert owner(begin[c]) == c and owner(begin[c + 1] - 1) == c
    for tile in range(nt):
        first, last = owner(tile * kbt), owner(tile * kbt + kbt - 1)
        assert 1 <= last - first + 1 <= slots
    assert jb.lib().jsm_linear_packed_bytes(N, K, paired) == U * 16384
