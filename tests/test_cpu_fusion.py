"""The IR fusion pass on its own (no GPU): which lines of a program it rewrites, and — more
important — every condition under which it must leave a program exactly as it is.

The positive cases are the op chains the reference's Python front end emits for RMSNorm and
softmax (tests/golden/frontend_ir/chains__*.ir, recorded from the unmodified front end), followed
by the deltensor lines a caller that tracks lifetimes appends for the chain's temporaries.
"""
from pathlib import Path

import pytest

from deepx_b200.executor import plan_fusion

GOLDEN = Path(__file__).resolve().parent / "golden" / "frontend_ir"
F = "tensor<float32>"


def chain_lines(name):
    return [l for l in (GOLDEN / name).read_text().splitlines() if l.strip()]


def with_deletes(lines, temps):
    return lines + [f"deltensor () -> ({F}:{t})" for t in temps]


RMS_TEMPS = ["48", "49", "50", "51", "52", "53", "54", "56"]     # 47 is x.float(), 55 the reshaped weight, 57 the output
SOFTMAX_TEMPS = ["58", "59", "60", "61", "62", "63", "64"]       # 65 is the output


def kinds(verdicts):
    return [v.split(" ")[0] for v in verdicts]


def test_frontend_rmsnorm_chain_becomes_one_op():
    lines = with_deletes(chain_lines("chains__rmsnorm_forward.ir"), RMS_TEMPS)
    n, v = plan_fusion("\n".join(lines))
    assert n == 1
    fused = [x for x in v if x.startswith("fused")]
    assert fused == [f"fused 0 rmsnorm({F}:45, {F}:55, var<float32>:8, var<float32>:1e-06)->({F}:57)"]
    k = kinds(v)
    # 9 of the 10 chain ops (the last became the fused op), 8 newtensor and 8 deltensor lines no longer run
    assert k.count("absorbed") == 9 + 8 + 8
    for line, kind in zip(lines, k):
        name = line.split("(")[0].strip()
        if name in ("arange", "constant", "todtype", "reshape", "divscalar", "subscalar") and kind != "run":
            assert name == "divscalar" and ":49" in line, line  # the only absorbed one of these is the chain's own divscalar
    # the output's newtensor, the x.float() copy and the weight reshape still run
    assert k[lines.index(next(l for l in lines if l.startswith("todtype")))] == "run"
    assert all(k[i] == "run" for i, l in enumerate(lines) if l.startswith("newtensor") and (":57)" in l or ":55)" in l or ":47)" in l))


def test_frontend_softmax_chain_becomes_one_op():
    lines = with_deletes(chain_lines("chains__softmax.ir"), SOFTMAX_TEMPS)
    n, v = plan_fusion("\n".join(lines))
    assert n == 1
    assert [x for x in v if x.startswith("fused")] == [f"fused 0 softmax({F}:45)->({F}:65)"]
    assert kinds(v).count("absorbed") == 7 + 7 + 7


def test_both_chains_in_one_program():
    rms = with_deletes(chain_lines("chains__rmsnorm_forward.ir"), RMS_TEMPS)
    sm = [l for l in chain_lines("chains__softmax.ir")[9:]]  # skip the shared setup
    n, v = plan_fusion("\n".join(rms + with_deletes(sm, SOFTMAX_TEMPS)))
    assert n == 2 and len([x for x in v if x.startswith("fused")]) == 2


def test_without_deletes_nothing_is_fused():
    """The front end of today never deletes its temporaries: they stay visible, so the chain must run as it is."""
    for name in ("chains__rmsnorm_forward.ir", "chains__softmax.ir"):
        lines = chain_lines(name)
        n, v = plan_fusion("\n".join(lines))
        assert n == 0 and set(kinds(v)) == {"run"}


def small_rms(sq="mul", extra_mid=None, extra_end=None, axis="2", keep="true", dtype="float32", weight=True, numer="1",
              deletes=("sq", "v", "vb", "y", "wb"), news=("sq", "v", "vb", "y", "wb", "out")):
    f = f"tensor<{dtype}>"
    shapes = {"sq": "4 6 8", "v": "4 6 1", "vb": "4 6 8", "y": "4 6 8", "wb": "4 6 8", "out": "4 6 8"}
    p = [f"newtensor(vector<int32>:[{shapes[n]}])->({f}:{n})" for n in news]
    p.append(f"mul({f}:x, {f}:x)->({f}:sq)" if sq == "mul" else f"powscalar({f}:x, var<int32>:2)->({f}:sq)")
    p.append(f"sum({f}:sq, vector<int32>:[{axis}], var<bool>:{keep})->({f}:v)")
    p.append(f"divscalar({f}:v, var<float32>:8)->({f}:v)")
    p.append(f"addscalar({f}:v, var<float32>:1e-6)->({f}:v)")
    if extra_mid:
        p.append(extra_mid)
    p.append(f"sqrt({f}:v)->({f}:v)")
    p.append(f"rdivscalar(var<float32>:{numer}, {f}:v)->({f}:v)")
    p.append(f"broadcastTo({f}:v, vector<int32>:[4 6 8])->({f}:vb)")
    p.append(f"mul({f}:x, {f}:vb)->({f}:y)")
    if weight:
        p.append(f"broadcastTo({f}:w, vector<int32>:[4 6 8])->({f}:wb)")
        p.append(f"mul({f}:y, {f}:wb)->({f}:out)")
    if extra_end:
        p.append(extra_end)
    p += [f"deltensor()->({f}:{n})" for n in deletes]
    return "\n".join(p)


EXISTING = "x float32 4 6 8\nw float32 8"


def test_hand_written_chain_in_place_vector_steps():
    """The benchmark's form of the chain: x*x and one [.,.,1] tensor updated in place."""
    n, v = plan_fusion(small_rms(), EXISTING)
    assert n == 1
    assert [x for x in v if x.startswith("fused")] == [f"fused 0 rmsnorm({F}:x, {F}:w, var<float32>:8, var<float32>:1e-6)->({F}:out)"]
    n, v = plan_fusion(small_rms(sq="pow"), EXISTING)
    assert n == 1


def test_chain_without_weight():
    prog = small_rms(weight=False, deletes=("sq", "v", "vb"), news=("sq", "v", "vb", "y"))
    n, v = plan_fusion(prog, EXISTING)
    assert n == 1
    assert [x for x in v if x.startswith("fused")] == [f"fused 0 rmsnorm({F}:x, var<float32>:8, var<float32>:1e-6)->({F}:y)"]


@pytest.mark.parametrize("why,prog,existing", [
    ("temporaries not deleted", small_rms(deletes=()), EXISTING),
    ("one temporary of the front part not deleted", small_rms(deletes=("sq", "v", "y", "wb")), EXISTING),
    ("temporary read by another op", small_rms(extra_end=f"add({F}:vb, {F}:x)->({F}:out)"), EXISTING),
    ("temporary existed before the program", small_rms(), EXISTING + "\nvb float32 4 6 8"),
    ("input rewritten under the chain", small_rms(extra_mid=f"addscalar({F}:x, var<float32>:1)->({F}:x)"), EXISTING),
    ("input deleted under the chain", small_rms(extra_mid=f"deltensor()->({F}:x)"), EXISTING),
    ("reduction not over the last axis", small_rms(axis="1"), EXISTING),
    ("keepdims false", small_rms(keep="false"), EXISTING),
    ("numerator is not 1", small_rms(numer="2"), EXISTING),
    ("integer tensors", small_rms(dtype="int32"), "x int32 4 6 8\nw int32 8"),
    ("input of unknown shape", small_rms(), "w float32 8"),
    ("input shape differs from the broadcast target", small_rms(), "x float32 4 6 16\nw float32 8"),
    ("dtype of a temporary differs", small_rms().replace("newtensor(vector<int32>:[4 6 1])->(tensor<float32>:v)", "newtensor(vector<int32>:[4 6 1])->(tensor<float64>:v)"), EXISTING),
])
def test_left_alone(why, prog, existing):
    n, v = plan_fusion(prog, existing)
    assert n == 0, why
    assert set(kinds(v)) == {"run"}, why


def test_front_part_fuses_when_only_the_weight_step_is_kept():
    """wb stays alive, so the weight multiply must run as it is; the part up to y still becomes one op."""
    prog = small_rms(deletes=("sq", "v", "vb", "y"))
    n, v = plan_fusion(prog, EXISTING)
    assert n == 1
    assert [x for x in v if x.startswith("fused")] == [f"fused 0 rmsnorm({F}:x, var<float32>:8, var<float32>:1e-6)->({F}:y)"]
    lines = prog.splitlines()
    for tail in (f"broadcastTo({F}:w, vector<int32>:[4 6 8])->({F}:wb)", f"mul({F}:y, {F}:wb)->({F}:out)", f"deltensor()->({F}:y)"):
        assert v[lines.index(tail)] == "run"


def test_weight_that_is_not_one_row_keeps_its_multiply():
    """w [6,8] broadcast to [4,6,8] varies along axis 1: not the row-weight of the fused op."""
    n, v = plan_fusion(small_rms(), "x float32 4 6 8\nw float32 6 8")
    assert n == 1
    assert [x for x in v if x.startswith("fused")] == [f"fused 0 rmsnorm({F}:x, var<float32>:8, var<float32>:1e-6)->({F}:y)"]


def test_numeral_tensor_names_do_not_collide_with_scalars():
    """The front end numbers its tensors; `var<int32>:8` in divscalar is not a use of tensor 8."""
    prog = small_rms().replace(":vb", ":8")
    n, _ = plan_fusion(prog, EXISTING)
    assert n == 1


def test_short_and_unrelated_programs_pass_through():
    n, v = plan_fusion(f"add({F}:a, {F}:b)->({F}:c)\nmul({F}:a, {F}:b)->({F}:c)", "a float32 4\nb float32 4\nc float32 4")
    assert n == 0 and v == ["run", "run"]
    lines = [f"mul({F}:a, {F}:b)->({F}:c)"] * 12
    n, v = plan_fusion("\n".join(lines), "a float32 4\nb float32 4\nc float32 4")
    assert n == 0 and set(v) == {"run"}


def test_parse_error_is_reported():
    with pytest.raises(ValueError):
        plan_fusion("this is not IR\n" * 9)
