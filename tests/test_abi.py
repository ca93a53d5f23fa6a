"""The C-ABI library: loads, exports every declared symbol, and its host-only functions
(no GPU needed) agree with the reference's host code through the golden fixtures."""
import ctypes as C
import json
import re
from pathlib import Path

import numpy as np

from turbogpt_b200 import Config, ConfigEx, OneCycle, StepRates
from turbogpt_b200 import bridge

ROOT = Path(__file__).resolve().parents[1]


def test_every_declared_symbol_is_exported(library):
    header = (ROOT / "include" / "turbogpt_b200.h").read_text()
    declared = set(re.findall(r"\b(tg_\w+)\s*\(", header))
    assert len(declared) >= 37
    for name in declared:
        assert hasattr(library, name), name
    assert {"tg_" + n for n in bridge.EXPORTS} <= declared
    assert {"tg_ex_" + n for n in bridge.EXTENSIONS} <= declared


def test_struct_layouts(library, golden):
    sizes = json.loads((golden / "ref_host.json").read_text())["sizes"]
    assert C.sizeof(Config) == sizes["Config"] == 72
    assert C.sizeof(OneCycle) == sizes["OneCycle"] == 48
    assert C.sizeof(StepRates) == sizes["StepRates"] == 8
    ex = ConfigEx.reference(Config())
    assert ex.struct_size == C.sizeof(ConfigEx) == 256
    assert (ex.width, ex.heads, ex.hidden, ex.world) == (16, 4, 48, 1)


def test_onecycle_point_matches_reference_bits(library, golden):
    for total, step, multiplier, momentum in json.loads((golden / "ref_host.json").read_text())["onecycle"]:
        rates = StepRates()
        assert library.tg_onecycle_point(C.byref(OneCycle(total)), step, C.byref(rates)) == 0
        assert np.float32(rates.multiplier).view(np.uint32) == multiplier
        assert np.float32(rates.momentum).view(np.uint32) == momentum
    rates = StepRates()
    assert library.tg_onecycle_point(C.byref(OneCycle(8)), 8, C.byref(rates)) < 0
    assert b"Invalid OneCycle" in library.tg_error()


def test_layout_and_initial_weights_match_reference(library, golden):
    h = json.loads((golden / "ref_host.json").read_text())
    for depth in (4, 8):
        ex = ConfigEx.reference(Config(depth=depth))
        assert library.tg_ex_parameter_count(C.byref(ex)) == h["parameter_count"][str(depth)]
    ex = ConfigEx.reference(Config(depth=4))
    layout = bridge.parameter_layout(ex)
    offsets = [o for o, _, _ in layout]
    assert offsets[0] == h["layout4"]["embedding"] and offsets[2] == h["layout4"]["l0_qkv"]
    assert offsets[-2] == h["layout4"]["final_norm"] and offsets[-1] == h["layout4"]["head"]
    w = bridge.initialize_weights(ex)
    assert len(w) == h["init_weights"]["count"]
    for index, bits in h["init_weights"]["first"]:
        assert int(w[index:index + 1].view(np.uint32)[0]) == bits
    from oracle.indexing import hash_u64
    checksum = 0
    for bits in w.view(np.uint32):
        checksum = hash_u64(checksum ^ int(bits))
    assert checksum == int(h["init_weights"]["checksum"])


def test_scaled_architecture_layout(library):
    from oracle.model import Arch, specification
    ex = ConfigEx.gpt(Config(depth=12), 768, 12)
    assert library.tg_ex_parameter_count(C.byref(ex)) == 85169664
    spec = specification(Arch.gpt(12, 768, 12))
    layout = bridge.parameter_layout(ex)
    assert len(layout) == len(spec)
    offset = 0
    for (o, rows, cols), (_, shape) in zip(layout, spec):
        assert o == offset and (rows, cols) == (shape[0], shape[1] if len(shape) == 2 else 0)
        offset += int(np.prod(shape))


def test_bad_configurations_are_refused_with_messages(library):
    def refused(**kwargs):
        ex = ConfigEx.reference(Config())
        for k, v in kwargs.items():
            setattr(ex, k, v)
        assert library.tg_ex_parameter_count(C.byref(ex)) < 0
        return library.tg_error().decode()
    assert "struct_size" in refused(struct_size=12)
    assert "width" in refused(width=20)
    assert "world" in refused(world=2, rank=2)
    ex = ConfigEx.reference(Config(inflight=2))
    assert not library.tg_create_ex(C.byref(ex))
    assert "requires build.ps1 -Pipeline" in library.tg_error().decode()
    ex = ConfigEx.reference(Config(ns_steps=11))
    assert not library.tg_create_ex(C.byref(ex))
    assert "ns_steps must be 1..10" in library.tg_error().decode()
    assert not library.tg_create(C.byref(Config(batch=3)))
    assert "batch at least 4" in library.tg_error().decode()
