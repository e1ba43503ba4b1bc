"""Pins the CPU oracle (``oracle/``) before anything is checked against it.

Three anchors, none of which needs a GPU:

* the format specification's known-answer words and structural facts
  (reference docs/format-spec.md:231-238, :319-325; tests/test_pack.py:78-85, :125-142);
* golden vectors produced by importing the reference's own Python implementation
  (``tests/golden/make_golden.py``);
* the two restatements (numpy and C) against each other, and -- when it has been built from
  the reference checkout -- the reference's compiled CPU operators in ``oracle/_ref``.
"""

from __future__ import annotations

import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

from oracle import oracle as O

ROOT = Path(__file__).resolve().parent.parent
GOLDEN = np.load(ROOT / "tests" / "golden" / "golden_v1.npz")
NUM_CASES = len([k for k in GOLDEN.files if k.endswith("_spec")])


def same_bits(a: np.ndarray, b: np.ndarray) -> bool:
    if a.dtype == np.float32:
        return bool((a.view(np.uint32) == b.view(np.uint32)).all())
    return bool((a == b).all())


def test_three_bit_known_answer():
    q = (np.arange(32) % 8).astype(np.uint8)[None]
    expect = np.array([[0x88FAC688, 0xC688FAC6, 0xFAC688FA]], dtype=np.uint32)
    assert (O.np_pack(q, 3) == expect).all()
    assert (O.c_pack(q, 3) == expect).all()
    assert (GOLDEN["kat3_words"] == expect[0]).all()


def test_three_bit_straddlers_are_exactly_10_and_21():
    for restate in (O.np_pack, O.c_pack):
        straddlers = []
        for i in range(32):
            q = np.zeros((1, 32), dtype=np.uint8)
            q[0, i] = 7
            words = restate(q, 3)[0]
            if np.count_nonzero(words) == 2:
                straddlers.append(i)
        assert straddlers == [10, 21]


@pytest.mark.parametrize("bits,words", [(2, 8), (3, 12), (4, 16), (8, 32)])
def test_words_per_group_at_128(bits, words):
    assert O.geometry(bits, 128, 4096).words_per_group == words


def test_size_accounting_matches_the_spec_table():
    # docs/format-spec.md:659-664: [256, 512] at group 128, fp16 scale + offset
    for bits, expect in ((2, 36864), (3, 53248), (4, 69632), (8, 135168)):
        g = O.geometry(bits, 128, 512)
        assert 256 * (g.words_per_row * 4 + g.num_groups * 2 * 2) == expect


@pytest.mark.parametrize("bits", [2, 3, 4, 8])
@pytest.mark.parametrize("n", [1, 2, 3, 7, 8, 31, 32, 33, 37, 96, 127, 128, 129, 1023])
def test_pack_matches_reference_words(bits, n):
    codes = GOLDEN[f"pack_b{bits}_n{n}_codes"]
    words = GOLDEN[f"pack_b{bits}_n{n}_words"]
    assert (O.np_pack(codes, bits) == words).all()
    assert (O.c_pack(codes, bits) == words).all()
    assert (O.np_unpack(words, bits, n) == codes).all()
    assert (O.c_unpack(words, bits, n) == codes).all()


def test_group_independence():
    """Changing one group's codes changes only that group's words (tests/test_pack.py:96-122)."""
    rng = np.random.default_rng(3)
    for bits in (2, 3, 4, 8):
        g = O.geometry(bits, 128, 512)
        codes = rng.integers(0, 1 << bits, size=(2, 4, 128)).astype(np.uint8)
        base = O.c_pack(codes, bits)
        codes2 = codes.copy()
        codes2[:, 2] = ((codes2[:, 2].astype(np.int64) + 1) % (1 << bits)).astype(np.uint8)
        changed = O.c_pack(codes2, bits)
        assert (base[:, [0, 1, 3]] == changed[:, [0, 1, 3]]).all()
        assert base.shape[-1] == g.words_per_group


def _case(ci):
    rows, k, group, bits, m, with_off = (int(v) for v in GOLDEN[f"case{ci}_spec"])
    meta = str(GOLDEN[f"case{ci}_meta"])
    return dict(
        rows=rows, k=k, group=group, bits=bits, m=m, meta=meta,
        packed=GOLDEN[f"case{ci}_packed"], scales=GOLDEN[f"case{ci}_scales"],
        offsets=GOLDEN[f"case{ci}_offsets"] if with_off else None,
        dequant=GOLDEN[f"case{ci}_dequant"], dequant_f32=GOLDEN[f"case{ci}_dequant_f32"],
        x=GOLDEN[f"case{ci}_x"], x_tag=str(GOLDEN[f"case{ci}_x_tag"]), y32=GOLDEN[f"case{ci}_y32"],
        geom=O.geometry(bits, group, k),
    )


@pytest.mark.parametrize("ci", range(NUM_CASES))
def test_dequant_is_bit_exact_against_the_reference(ci):
    c = _case(ci)
    for restate in (O.np_dequant, O.c_dequant):
        got = restate(c["packed"], c["scales"], c["offsets"], c["meta"], c["geom"])
        assert same_bits(got, c["dequant"]), restate.__name__
        got32 = restate(c["packed"], c["scales"], c["offsets"], c["meta"], c["geom"], "f32")
        assert same_bits(got32, c["dequant_f32"]), restate.__name__


@pytest.mark.parametrize("ci", range(NUM_CASES))
def test_gemv_matches_the_reference_test_oracle(ci):
    c = _case(ci)
    want = c["y32"]
    scale = np.abs(want).max() + 1e-30
    for restate in (O.np_gemv, O.c_gemv):
        got = restate(c["x"], c["x_tag"], c["packed"], c["scales"], c["offsets"], c["meta"], c["geom"])
        # the reference sums in fp32 (torch matmul), the oracle in fp64: reassociation noise only
        assert np.abs(got - want).max() / scale < 2e-6, restate.__name__


@pytest.mark.parametrize("ci", range(NUM_CASES))
def test_reference_torch_path_is_within_its_own_tolerance(ci):
    """The reference's torch path rounds the weight to the activation dtype first; it sits
    ~2.5e-3 from the fp32 oracle in bf16, inside the 2e-2 its tests allow."""
    c = _case(ci)
    y = O.to_f32(GOLDEN[f"case{ci}_y_torch_path"], c["x_tag"])
    want = c["y32"]
    assert np.allclose(y, want, rtol=2e-2, atol=2e-2 * max(1.0, float(np.abs(want).max())))


def test_float_converters_agree_with_numpy_and_torch():
    import torch

    rng = np.random.default_rng(0)
    vals = np.concatenate([
        rng.standard_normal(4096).astype(np.float32) * 10.0 ** rng.integers(-8, 5, 4096),
        np.array([0.0, -0.0, 65504.0, 65519.9, 65520.0, 1e-8, 5.96e-8, 2.98e-8, 2.99e-8, np.inf, -np.inf],
                 dtype=np.float32),
    ]).astype(np.float32)
    lib = O.lib()
    import ctypes

    for tag, tdt in (("f16", torch.float16), ("bf16", torch.bfloat16)):
        out = np.empty(vals.shape, dtype=np.uint16)
        lib.dqo_convert_from_f32(vals.ctypes.data_as(ctypes.c_void_p), out.ctypes.data_as(ctypes.c_void_p),
                                 ctypes.c_int64(vals.size), O.DTYPE_TAGS[tag])
        want = torch.from_numpy(vals).to(tdt).view(torch.int16).numpy().view(np.uint16)
        assert (out == want).all(), tag
        assert (O.from_f32(vals, tag) == want).all(), tag
        back = np.empty(vals.shape, dtype=np.float32)
        lib.dqo_convert_to_f32(out.ctypes.data_as(ctypes.c_void_p), back.ctypes.data_as(ctypes.c_void_p),
                               ctypes.c_int64(vals.size), O.DTYPE_TAGS[tag])
        assert same_bits(back, O.to_f32(out, tag))


def test_moe_restatements_agree():
    rng = np.random.default_rng(5)
    hidden, inter, experts, topk, tokens = 256, 128, 4, 2, 3
    def bank(rows, k, bits):
        g = O.geometry(bits, 128, k)
        packed = rng.integers(0, 2**32, size=(rows, g.words_per_row), dtype=np.uint64).astype(np.uint32)
        scales = O.from_f32(rng.uniform(0.005, 0.02, size=(rows, g.num_groups)).astype(np.float32), "f16")
        offsets = O.from_f32(-(1 << (bits - 1)) * O.to_f32(scales, "f16"), "f16")
        return (packed, scales, offsets, "f16", g)
    gate_up = bank(experts * 2 * inter, hidden, 3)
    down = bank(experts * hidden, inter, 4)
    x = O.from_f32(rng.standard_normal((tokens, hidden)).astype(np.float32), "bf16")
    ids = np.stack([rng.permutation(experts)[:topk] for _ in range(tokens)]).astype(np.int32)
    w = rng.uniform(0.1, 1.0, size=(tokens, topk)).astype(np.float32)
    a = O.np_moe(x, "bf16", ids, w, gate_up, down, inter=inter, num_experts=experts)
    b = O.c_moe(x, "bf16", ids, w, gate_up, down, inter=inter, num_experts=experts)
    assert np.abs(a - b).max() <= 2e-5 * np.abs(a).max()


def test_against_the_reference_compiled_cpu_operators_when_built():
    """``oracle/_ref`` is the reference's own bindings.cpp compiled in place.  It registers the
    ``dynquant::`` operator namespace, so it is exercised in a child process."""
    ref = ROOT / "oracle" / "_ref" / "libdynquant_ref_cpu.so"
    if not ref.exists():
        pytest.skip("oracle/_ref not built (needs the reference checkout)")
    script = f"""
import sys, numpy as np, torch
sys.path.insert(0, {str(ROOT)!r})
torch.ops.load_library({str(ref)!r})
from oracle import oracle as O
g = np.load({str(ROOT / 'tests' / 'golden' / 'golden_v1.npz')!r})
dt = {{'f16': torch.float16, 'bf16': torch.bfloat16, 'f32': torch.float32}}
def t(a, tag):
    return torch.from_numpy(a.view(np.int16).copy()).view(dt[tag]) if tag != 'f32' else torch.from_numpy(a.copy())
n = len([k for k in g.files if k.endswith('_spec')])
for ci in range(n):
    rows, k, group, bits, m, with_off = (int(v) for v in g[f'case{{ci}}_spec'])
    meta = str(g[f'case{{ci}}_meta'])
    geom = O.geometry(bits, group, k)
    packed = torch.from_numpy(g[f'case{{ci}}_packed'].view(np.int32).copy())
    scales = t(g[f'case{{ci}}_scales'], meta)
    offsets = t(g[f'case{{ci}}_offsets'], meta) if with_off else None
    dense = torch.ops.dynquant.dequant(packed, scales, offsets, bits, geom.group_values, k)
    mine = O.c_dequant(g[f'case{{ci}}_packed'], g[f'case{{ci}}_scales'], g[f'case{{ci}}_offsets'] if with_off else None, meta, geom)
    ref_bits = dense.view(torch.int16).numpy().view(np.uint16) if meta != 'f32' else dense.numpy()
    if meta == 'f32':
        assert np.allclose(ref_bits, mine, rtol=1e-6, atol=1e-6), ci
    else:
        assert (ref_bits == mine).all(), ci
print('ok')
"""
    res = subprocess.run([sys.executable, "-c", script], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0 and "ok" in res.stdout, res.stderr[-2000:]
