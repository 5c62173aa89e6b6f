"""The compact-schedule adapter (veritac_b200/specializations/gemmini_gemm/schedule_ir.py) against what the
reference's adapter returned for the same expressions and programs (values, expansions, refusal texts), and
against the cases of the reference's own tests/test_gemmini_schedule_ir.py."""
import hashlib
import json

import pytest

from veritac_b200.specializations.gemmini_gemm import backend as g
from veritac_b200.specializations.gemmini_gemm import schedule_ir as ir
from veritac_b200.specializations.gemmini_gemm.schedule_ir import ScheduleError, expand_program, expression


def sha(obj):
    return hashlib.sha256(json.dumps(obj, sort_keys=True).encode()).hexdigest()


def loop(stop, body, start=0, step=1):
    return {"for": "i", "start": start, "stop": stop, "step": step, "body": body}


def test_expressions_like_the_reference(golden_schedule_ir):
    env = golden_schedule_ir["bindings"]
    for e in golden_schedule_ir["expressions"]:
        if "error" in e:
            with pytest.raises(ScheduleError) as info:
                expression(e["text"], env)
            assert str(info.value) == e["error"], e["text"]
        else:
            v = expression(e["text"], env)
            assert v == e["value"] and (type(v) is bool) == e["is_bool"], e["text"]


def test_programs_like_the_reference(golden_schedule_ir):
    for p in golden_schedule_ir["programs"]:
        if "error" in p:
            with pytest.raises(ScheduleError) as info:
                expand_program(p["program"], p["constants"], **p["limits"])
            assert str(info.value) == p["error"], p["name"]
            continue
        out = expand_program(p["program"], p["constants"], **p["limits"])
        assert len(out) == p["expanded_len"] and sha(out) == p["expanded_sha256"], p["name"]
        if "expanded" in p:
            assert out == p["expanded"]


def test_loop_form_of_the_baseline_is_the_generator_stream(golden_schedule_ir):
    p = golden_schedule_ir["programs"][0]
    out = expand_program(p["program"], p["constants"])
    assert out == g.serialize_commands(g.gen_commands(p["plan"]))


def test_negative_steps_follow_range():
    for start, stop, step in ((5, -2, -2), (2, 5, -1), (-3, -6, -2), (5, 0, -3)):
        out = expand_program([loop(stop, [{"kind": "x", "i": {"expr": "i"}}], start, step)], {})
        assert [x["i"] for x in out] == list(range(start, stop, step))


def test_nothing_is_executed_and_nothing_rebound():
    for text in ("__import__('os').system('true')", "M.bit_length()", "2 ** 10000000", "M[0]", "1 / 2", "True + 1",
                 "1 // 0", "1 << 99", "0 if True else int('1')", "0 if True else missing"):
        with pytest.raises(ScheduleError):
            expression(text, {"M": 32})
    with pytest.raises(ScheduleError):
        expand_program([loop(2, [])], {"i": 1})
    assert expression("i > 0", {"i": 1}) is True
    assert expression("10 if i == 0 else 20", {"i": 0}) == 10
    with pytest.raises(ScheduleError):
        expand_program([loop(True, [])], {})
    for limits in ({"max_commands": 0}, {"max_iterations": -1}, {"max_depth": True}):
        with pytest.raises(ScheduleError):
            expand_program([], {}, **limits)
    assert ir.expression("0xA0000000 if i == 0 else 0xE0000000", {"i": 3}) == 0xE0000000
