"""The C-ABI library loads, exports every symbol the public header declares and validates
its arguments before touching the GPU (no kernel is launched in this file)."""
import ctypes
import os
import re

from trinix_b200 import _lib

HEADER = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "include",
                      "trinix_b200.h")
I64x3 = _lib.I64x3


def _declared():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(trx_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound(lib):
    names = _declared()
    assert len(names) >= 11
    for n in names:
        assert hasattr(lib, n), f"{n} declared in the header but not exported"
        assert n in _lib.SIGNATURES, f"{n} has no ctypes signature"
    assert sorted(_lib.SIGNATURES) == names


def test_version_and_status_strings(lib):
    assert lib.trx_version() == 1
    assert lib.trx_status_string(0) == b"ok"
    for code in range(-9, 0):
        assert lib.trx_status_string(code) not in (b"ok", b"unknown status code")
    assert lib.trx_status_string(-99) == b"unknown status code"
    assert lib.trx_attn_workspace_bytes() >= 16


def test_rowwise_argument_validation(lib):
    P = ctypes.c_void_p
    one = P(16)
    assert lib.trx_rmsnorm_fwd(None, one, one, None, 4, 8, 8, 8, 1e-6, 2, 2, None) == -1
    assert lib.trx_rmsnorm_fwd(one, one, one, None, 4, 8, 8, 8, 1e-6, 7, 2, None) == -2
    assert lib.trx_rmsnorm_fwd(one, one, one, None, 4, 0, 8, 8, 1e-6, 2, 2, None) == -3
    assert lib.trx_rmsnorm_fwd(one, one, one, None, 4, 8, 4, 8, 1e-6, 2, 2, None) == -5
    assert lib.trx_rmsnorm_fwd(None, None, None, None, 0, 8, 8, 8, 1e-6, 2, 2, None) == 0  # no rows
    assert lib.trx_layernorm_fwd(one, None, None, None, None, None, 4, 8, 8, 8, 1e-5, 2, 2, None) == -1
    assert lib.trx_quant_rowwise_i8(one, None, one, 4, 8, 8, 8, 2, None) == -1
    assert lib.trx_quant_rowwise_i8(one, one, one, 4, 8, 8, 4, 2, None) == -5
    assert lib.trx_dequant_rowwise_i8(one, one, one, 4, 8, 8, 8, 9, None) == -2
    assert lib.trx_rmsnorm_quant_i8(one, None, one, one, 4, 8, 8, 8, 1e-6, 2, 2, None) == -1
    assert lib.trx_glu_fwd(one, one, one, 4, 8, 8, 8, 8, 5, 2, None) == -6
    assert lib.trx_glu_fwd(one, one, one, 4, 8, 8, 4, 8, 0, 2, None) == -5


def test_rope_and_attention_argument_validation(lib):
    P = ctypes.c_void_p
    one = P(4096)
    st = I64x3(64, 8, 8)
    assert lib.trx_rope_fwd(one, one, one, one, one, one, 1, 4, 1, 1, 7, st, st, st, st, 8, 0, 2, 0,
                            None) == -3  # odd head_dim
    assert lib.trx_rope_fwd(one, one, one, one, one, one, 1, 4, 1, 1, 8, st, st, st, st, 8, 1, 2, 0,
                            None) == -2  # fp16 tables with bf16 activations
    # stride arrays are passed through correctly: a negative entry in the LAST array is caught
    bad = I64x3(64, 8, -1)
    assert lib.trx_rope_fwd(one, one, one, one, one, one, 1, 4, 1, 1, 8, st, st, st, bad, 8, 0, 2, 0,
                            None) == -5
    assert lib.trx_rope_fwd(one, one, None, one, one, one, 1, 4, 1, 1, 8, st, st, st, st, 8, 0, 2, 0,
                            None) == -1
    ws = P(4096)
    a = (one, one, one, one, None, None)
    assert lib.trx_attn_fwd(*a, 1, 8, 8, 4, 3, 128, st, st, st, st, 1.0, 0, -1, -1, 2, ws, 256,
                            None) == -3  # Hq % Hk
    assert lib.trx_attn_fwd(*a, 1, 8, 8, 4, 2, 96, st, st, st, st, 1.0, 0, -1, -1, 2, ws, 256,
                            None) == -6  # head_dim
    assert lib.trx_attn_fwd(*a, 1, 8, 8, 4, 2, 128, st, st, st, st, 1.0, 0, -1, -1, 0, ws, 256,
                            None) == -2  # fp32
    assert lib.trx_attn_fwd(*a, 1, 8, 8, 4, 2, 128, st, st, st, st, 1.0, 0, 4, -1, 2, ws, 256,
                            None) == -3  # half-specified window
    assert lib.trx_attn_fwd(*a, 1, 8, 8, 4, 2, 128, st, st, st, st, 1.0, 0, -1, -1, 2, None, 0,
                            None) == -9  # workspace
    assert lib.trx_attn_fwd(*a, 1, 8, 8, 4, 2, 128, st, st, st, st, 1.0, 0, -1, -1, 2, ws, 8,
                            None) == -9
    assert lib.trx_attn_fwd(*a, 0, 8, 8, 4, 2, 128, st, st, st, st, 1.0, 0, -1, -1, 2, ws, 256,
                            None) == 0  # empty batch


def test_status_entry_point_validates_without_a_device(lib):
    P = ctypes.c_void_p
    word = ctypes.c_uint(0)
    assert lib.trx_attn_status(None, ctypes.byref(word), None) == -1
    assert lib.trx_attn_status(P(4096), None, None) == -1
    word.value = 4  # a failure seen by an earlier copy: reported, nothing enqueued
    assert lib.trx_attn_status(P(4096), ctypes.byref(word), None) == -8
    assert word.value == 4


def test_two_host_threads_on_first_use(lib):
    """The library keeps a few per-device caches (driver entry point, occupancy answers, the
    dynamic shared-memory attribute). Two host threads that make their first calls at the same
    moment must get the same, correct status codes; the validation-only paths below reach the
    shared state behind `make_map` without launching anything."""
    import threading
    P = ctypes.c_void_p
    one, ws, st = P(4096), P(4096), I64x3(64, 8, 8)
    a = (one, one, one, one, None, None)
    results = [[], []]
    start = threading.Barrier(2)

    def work(slot):
        start.wait()
        for _ in range(200):
            results[slot].append((
                lib.trx_attn_fwd(*a, 1, 8, 8, 4, 3, 128, st, st, st, st, 1.0, 0, -1, -1, 2, ws, 256,
                                 None),
                lib.trx_attn_fwd(*a, 1, 8, 8, 4, 2, 128, I64x3(64, 8, 3), st, st, st, 1.0, 0, -1,
                                 -1, 2, ws, 256, None),   # reaches make_map: stride not 16-byte
                lib.trx_rmsnorm_fwd(one, one, one, None, 4, 8, 4, 8, 1e-6, 2, 2, None),
                lib.trx_attn_fwd_static_scratch(*a, 1, 8, 8, 4, 2, 96, st, st, st, st, 1.0, 0, -1,
                                                -1, 2, None, None),
            ))

    ts = [threading.Thread(target=work, args=(i,)) for i in range(2)]
    for t in ts:
        t.start()
    for t in ts:
        t.join()
    assert results[0] == results[1]
    first = results[0][0]
    assert first[0] == -3 and first[2] == -5 and first[1] in (-4, -7) and first[3] in (-6, -7)
    assert all(r == first for r in results[0])


def test_product_does_not_import_the_oracle():
    """No module of the product package may reach into oracle/ or the scratch folder."""
    pkg = os.path.join(os.path.dirname(HEADER), "..", "trinix_b200")
    for root, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh")):
                src = open(os.path.join(root, f)).read()
                assert not re.search(r"\boracle\b", src), f
                assert not re.search(r"[\"'/]_work\b", src), f
