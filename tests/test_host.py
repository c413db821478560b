"""CPU tests of the host side: the C ABI library loads and exports what the
header declares, plans in the reference's JSON format are parsed, validated and
lowered without a GPU, the planner follows the reference's config precedence
and task-merging rules, and the multi-rank bootstrap plumbing works over gloo."""
import ctypes
import glob
import json
import os
import re
import subprocess
import sys

import numpy as np
import pytest

import ark_b200 as ark
from ark_b200.executor import LIB_PATH, lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    hdr = open(os.path.join(ROOT, "include", "ark_b200.h")).read()
    names = sorted(n for n in set(re.findall(r"\b(arkb_[a-z_]+)\s*\(", hdr)) if n not in ("arkb_status", "arkb_allgather_fn"))
    assert len(names) >= 20
    L = ctypes.CDLL(LIB_PATH)
    for n in names:
        assert hasattr(L, n), f"{n} is declared in include/ark_b200.h but not exported"
    assert ark.version().count(".") == 2


def _ffn_plan(num_sm=148):
    ark.init()
    x, w1, w2 = ark.tensor([128, 1024], ark.fp16), ark.tensor([1024, 4096], ark.fp16), ark.tensor([4096, 1024], ark.fp16)
    with ark.PlannerContext(sync=False):
        h = ark.relu(ark.matmul(x, w1))
    y = ark.matmul(h, w2)
    return ark.Planner(0, num_sm=num_sm).plan()


def test_plan_has_reference_fields_and_merges_unsynced_ops():
    plan = _ffn_plan().plan
    for k in ("Rank", "WorldSize", "Architecture", "NumProcessors", "NumWarpsPerProcessor", "TaskInfos", "ProcessorGroups"):
        assert k in plan
    assert plan["Architecture"] == "CUDA_100"
    assert [len(t["Ops"]) for t in plan["TaskInfos"]] == [2, 1]  # matmul+relu share a task (Sync=false)
    op = plan["TaskInfos"][0]["Ops"][0]
    assert op["Type"] == "Matmul" and op["Args"]["TransposeOther"] == {"BOOL": False}
    assert op["Config"]["TileShapeMNK"] == [128, 256, 64] and op["Config"]["NumTasks"] == 16
    t = op["ReadTensors"][0]
    assert set(t) == {"Id", "DataType", "Shape", "Strides", "Offsets", "PaddedShape", "Buffer"}
    assert set(t["Buffer"]) == {"Id", "Rank", "SendTags", "RecvTags"}


def test_plan_lowering_fuses_activation_and_places_barriers():
    plan = _ffn_plan()
    n_stages, arena, procs = ark.plan_check(str(plan))
    text = ark.plan_dump(str(plan))
    # X W1 with the ReLU in its epilogue; the second matmul (128 rows, 8 column tiles, K = 4096) runs swapped with K
    # cut into ranges so that every SM streams weights, then the sum of the partials
    assert procs == 148 and n_stages == 5
    assert "act=1" in text and text.count("sync group") == 2 and "swapped" in text and "split-K sum" in text
    assert arena >= (128 * 1024 + 2 * 1024 * 4096 + 128 * 4096 + 128 * 1024) * 2


def test_barrier_rule_between_processor_groups():
    """Disjoint processor groups run without a barrier; overlapping ones get one (ark/codegen.cpp:109-158)."""
    ark.init()
    a, b = ark.tensor([64, 64], ark.fp32), ark.tensor([64, 64], ark.fp32)
    with ark.PlannerContext(processor_range=[0, 8]):
        c = ark.add(a, b)
    with ark.PlannerContext(processor_range=[8, 16]):
        d = ark.mul(a, b)
    with ark.PlannerContext(processor_range=[0, 16]):
        e = ark.add(c, d)
    text = ark.plan_dump(str(ark.Planner(0, num_sm=148).plan()))
    lines = [l for l in text.strip().split("\n")[1:] if not l.startswith("arena=")]
    kinds = [("sync" if "sync group" in l else "op") for l in lines]
    assert kinds == ["op", "op", "sync", "op"]
    assert "[0,16) sync" in lines[2]


def test_config_precedence_context_over_rule_over_default():
    ark.init()
    a = ark.tensor([64, 64], ark.fp32)
    with ark.PlannerContext(config={"Tile": [2, 32]}):
        ark.exp(a)
    ark.relu(a)
    pl = ark.Planner(0, num_sm=148)
    pl.install_config_rule(lambda op, arch: json.dumps({"NumWarps": 2, "SramBytes": 0, "NumTasks": 7, "Tile": [4, 16]})
                           if json.loads(op)["Type"] == "Relu" else "")
    plan = pl.plan().plan
    assert plan["TaskInfos"][0]["Ops"][0]["Config"]["Tile"] == [2, 32]
    assert plan["TaskInfos"][1]["Ops"][0]["Config"]["Tile"] == [4, 16]


@pytest.mark.parametrize("mutate,err", [
    (lambda p: p.__setitem__("Rank", 3), ark.InvalidUsageError),
    (lambda p: p.pop("TaskInfos"), ark.PlanError),
    (lambda p: p["ProcessorGroups"][0].__setitem__("ProcessorRange", [0, 4096]), ark.PlanError),
    (lambda p: p["TaskInfos"][0]["Ops"][0].__setitem__("Type", "Conv9000"), ark.UnsupportedError),
    (lambda p: p["ProcessorGroups"][0]["ResourceGroups"][0]["TaskGroups"][0].__setitem__("TaskId", 77), ark.PlanError),
    (lambda p: p.__setitem__("NumProcessors", 500), ark.UnsupportedError),
])
def test_plan_errors(mutate, err):
    plan = _ffn_plan().plan
    mutate(plan)
    if plan.get("NumProcessors") == 500:
        plan["ProcessorGroups"][0]["ProcessorRange"] = [0, 500]
        plan["ProcessorGroups"][0]["ResourceGroups"][0]["ProcessorRange"] = [0, 500]
    with pytest.raises(err):
        ark.plan_check(json.dumps(plan))


def test_not_json_is_a_plan_error():
    with pytest.raises(ark.PlanError):
        ark.plan_check("{oops")


def test_model_errors():
    ark.init()
    a, b = ark.tensor([4, 8], ark.fp32), ark.tensor([5, 8], ark.fp32)
    with pytest.raises(ark.ModelError):
        ark.add(a, b)
    with pytest.raises(ark.ModelError):
        ark.matmul(a, b)
    with pytest.raises(ark.ModelError):
        ark.reduce_sum(a, axis=5)
    with pytest.raises(ark.ModelError):
        ark.tensor([1, 2, 3, 4, 5], ark.fp32)


def test_multi_rank_plan_lowering_all_reduce_and_send_recv():
    for algo_elems, expect in ((4096, "one-shot"), (4 * 1024 * 1024, "two-shot")):
        ark.init()
        ark.set_rank(1)
        ark.set_world_size(4)
        t = ark.tensor([algo_elems], ark.fp16)
        ark.all_reduce(t, 1, 4, output=t)
        text = ark.plan_dump(str(ark.Planner(0, num_sm=148).plan()))
        assert expect in text and "peer barrier" in text
    ark.init()
    ark.set_rank(0)
    ark.set_world_size(2)
    t = ark.tensor([1024], ark.fp16)
    s = ark.send(t, 1, tag=5)
    ark.send_done(s)
    r = ark.recv(ark.tensor([1024], ark.fp16), 1, tag=6)
    plan = ark.Planner(0, num_sm=148).plan()
    ops = [o for ti in plan.plan["TaskInfos"] for o in ti["Ops"]]
    assert ops[0]["WriteTensors"][0]["Buffer"]["Rank"] == 1
    assert ops[0]["WriteTensors"][0]["Buffer"]["RecvTags"] == [[-1, 5]]
    assert ops[0]["ReadTensors"][0]["Buffer"]["SendTags"] == [[1, 5]]
    ark.set_rank(0)
    ark.set_world_size(1)


def test_matmul_and_all_reduce_of_one_task_are_fused():
    """Planned as one task (Sync=false), a Matmul and the AllReduce of its result become: tiles stored into the summing
    rank's staging slots by the epilogue, then one sum-and-gather stage; otherwise matmul, then the two-shot collective."""
    from ark_b200.ffn import build_ffn
    for tokens, fused in ((1024, True), (256, False)):
        ark.init()
        ark.set_rank(1)
        ark.set_world_size(2)
        build_ffn(tokens, 512, 2048, ark.fp16, 1, 2)
        text = ark.plan_dump(str(ark.Planner(0, num_sm=148).plan()))
        assert ("tiles->peer slots" in text) == fused and ("sum of staging slots" in text) == fused
        assert ("two-shot" in text or "one-shot" in text) == (not fused)
        assert "peer barrier" in text
    ark.set_rank(0)
    ark.set_world_size(1)


def test_decode_layer_folds_small_operators_into_the_weight_streaming_matmuls():
    """One token per sequence: norm, gate*up and the residual adds ride in the matmul stages (planned as one task
    each), attention is one stage plus its merge; a prefill layer keeps them as stages of their own."""
    from ark_b200.llama import LlamaConfig, decoder_layer, layer_weights
    cfg = LlamaConfig(dim=4096, n_heads=32, n_kv_heads=32, ffn_dim=11008)
    ark.init()
    x, rope = ark.tensor([1, 4096], ark.fp16), ark.tensor([1, 1, 1, 128], ark.fp16)
    w = layer_weights(cfg, ark.fp16, 1)
    kc, vc = ark.tensor([1, 32, 2048, 128], ark.fp16), ark.tensor([1, 32, 2048, 128], ark.fp16)
    decoder_layer(x, w, cfg, 1, 1, 0, 1, rope=rope, k_cache=kc, v_cache=vc)
    text = ark.plan_dump(str(ark.Planner(0, num_sm=148).plan()))
    assert text.count("Matmul(gemv)") == 4 and text.count("<-rmsnorm") == 2 and text.count("+residual") == 2
    assert "<-mul" in text and "DecodeAttention" in text
    # the query's rotary embedding is applied by the attention stage while it loads q, and the attention's chunks are
    # merged by the output projection while it stages its activations: six compute stages and four barriers per layer
    assert "<-rope" in text and "<-attention merge" in text and "Rope rope" not in text and "merge of the chunks" not in text
    # W1 and W3 (same activations, same norm, same shape) are one weight-streaming stage over both matrices
    assert text.count("sync group") == 4 and len(text.splitlines()) == 11 and "(second matrix, act=0" in text, text
    assert "RMSNorm" not in text and " Add " not in text and " Mul " not in text
    ark.init()
    x, rope = ark.tensor([256, 4096], ark.fp16), ark.tensor([1, 256, 1, 128], ark.fp16)
    mask = ark.tensor([1, 1, 256, 256], ark.fp16)
    w = layer_weights(cfg, ark.fp16, 1)
    decoder_layer(x, w, cfg, 1, 256, 0, 1, rope=rope, mask=mask)
    text = ark.plan_dump(str(ark.Planner(0, num_sm=148).plan()))
    assert "Matmul(gemv)" not in text and text.count("RMSNorm") == 2 and "Softmax" in text


def test_causal_prefill_layer_lowers_to_one_attention_stage():
    """causal=True: no mask tensor, no transposes, no scores tensor; the attention block is one stage of 128-row units;
    its tensor-core instructions are per CTA, so the plan is not lowered for CTA pairs."""
    from ark_b200.llama import LlamaConfig, decoder_layer, layer_weights
    cfg = LlamaConfig(dim=8192, n_heads=8, n_kv_heads=1, ffn_dim=3584)   # one rank's share of the 70B shape at TP8
    ark.init()
    x, rope = ark.tensor([4 * 1024, 8192], ark.bf16), ark.tensor([1, 1024, 1, 128], ark.bf16)
    w = layer_weights(cfg, ark.bf16, 1)
    decoder_layer(x, w, cfg, 4, 1024, 0, 1, rope=rope, causal=True)
    text = ark.plan_dump(str(ark.Planner(0, num_sm=148).plan()))
    assert "PrefillAttention prefill_attention B=4 heads=8/1 rows=1024 keys=1024 causal bthd units=256" in text
    assert "Transpose" not in text and "Softmax" not in text and " pairs" not in text.splitlines()[0]
    # RoPE in the Q and K projections' epilogues, gate * up in W3's, the residual in W2's: no elementwise stage is left,
    # and W3 follows W1 without a barrier (same tiles on the same CTAs)
    assert text.count(" rope ") == 2 and "Rope" not in text and " Mul " not in text and " Add " not in text
    assert "*operand" in text and "+operand" in text
    lines = text.splitlines()
    w1 = next(i for i, l in enumerate(lines) if "act=4" in l)
    assert "*operand" in lines[w1 + 1]
    # shapes the stage does not take are refused when the model is built / lowered, not at run time
    ark.init()
    q, k = ark.tensor([1, 4, 256, 64], ark.fp16), ark.tensor([1, 4, 256, 64], ark.fp16)
    with pytest.raises(ark.ModelError):
        ark.prefill_attention(q, k, k)
    ark.init()
    q, k = ark.tensor([1, 4, 256, 128], ark.fp32), ark.tensor([1, 4, 256, 128], ark.fp32)
    ark.prefill_attention(q, k, k)
    with pytest.raises(ark.UnsupportedError):
        ark.plan_dump(str(ark.Planner(0, num_sm=148).plan()))
    with pytest.raises(ValueError):
        ark.init()
        cfg64 = LlamaConfig(dim=512, n_heads=8, n_kv_heads=8, head_dim=64, ffn_dim=1376)
        decoder_layer(ark.tensor([256, 512], ark.fp16), layer_weights(cfg64, ark.fp16, 1), cfg64, 1, 256, 0, 1, causal=True)


def test_tall_tiles_are_an_opt_in_of_the_one_cta_form(monkeypatch):
    """ARKB_TALL (off by default: measured slower) gives a CTA 256-row tiles as two halves over one B block; only
    without CTA pairs, and the ring then holds 32 KiB of A per slot."""
    def dump():
        ark.init()
        a, b = ark.tensor([2048, 4096], ark.fp16), ark.tensor([4096, 4096], ark.fp16)
        ark.matmul(a, b, transpose_other=True)
        return ark.plan_dump(str(ark.Planner(0, num_sm=148).plan())).splitlines()[1]
    assert " tall" not in dump() and "tile_n=256" in dump()            # pairs by default
    monkeypatch.setenv("ARKB_NO_PAIR", "1")
    assert " tall" not in dump() and "units=288" in dump() and "stages=4" in dump()
    monkeypatch.setenv("ARKB_TALL", "2")
    line = dump()
    assert " tall " in line and "units=144" in line and "stages=3" in line, line
    monkeypatch.delenv("ARKB_NO_PAIR")
    assert " tall" not in dump()                                        # never with pairs
    ark.init()


def test_prefill_attention_takes_a_mask_tensor():
    """The general form of the fused stage: an additive mask [B or 1, Hq or 1, Tq, Tkv]; wrong shapes are refused when
    the model is built, a mask of another type or with unaligned rows when the plan is lowered."""
    ark.init()
    q, k = ark.tensor([2, 4, 256, 128], ark.fp16), ark.tensor([2, 2, 384, 128], ark.fp16)
    ark.prefill_attention(q, k, k, 0.1, causal=False, mask=ark.tensor([2, 1, 256, 384], ark.fp16))
    text = ark.plan_dump(str(ark.Planner(0, num_sm=148).plan()))
    assert "PrefillAttention prefill_attention B=2 heads=4/2 rows=256 keys=384 +mask bhtd units=16" in text
    for shape in ([1, 1, 256, 256], [3, 1, 256, 384], [2, 2, 256, 384]):
        ark.init()
        q, k = ark.tensor([2, 4, 256, 128], ark.fp16), ark.tensor([2, 2, 384, 128], ark.fp16)
        with pytest.raises(ark.ModelError):
            ark.prefill_attention(q, k, k, 0.1, causal=False, mask=ark.tensor(shape, ark.fp16))
    ark.init()
    q, k = ark.tensor([1, 4, 256, 128], ark.fp16), ark.tensor([1, 4, 260, 128], ark.fp16)
    ark.prefill_attention(q, k, k, 0.1, causal=False, mask=ark.tensor([1, 1, 256, 260], ark.fp16))   # rows of 520 bytes
    with pytest.raises(ark.UnsupportedError):
        ark.plan_dump(str(ark.Planner(0, num_sm=148).plan()))
    ark.init()
    q, k = ark.tensor([1, 4, 256, 128], ark.fp16), ark.tensor([1, 4, 256, 128], ark.fp16)
    ark.prefill_attention(q, k, k, 0.1, causal=False, mask=ark.tensor([1, 1, 256, 256], ark.bf16))
    with pytest.raises(ark.UnsupportedError):
        ark.plan_dump(str(ark.Planner(0, num_sm=148).plan()))
    ark.init()


def test_narrow_prefill_projections_run_side_by_side():
    """At tensor-parallel degree 8 a rank's share of Wq, Wk and Wv is 512 columns: each runs on a third of the processors
    with wide tiles, no barrier between the three; the plan still keeps the barrier after the norm and before the
    attention stage. At degree 1 the projections keep the whole grid."""
    from ark_b200.llama import LlamaConfig, decoder_layer, layer_weights
    cfg = LlamaConfig(dim=4096, n_heads=32, n_kv_heads=32, ffn_dim=11008)
    for world in (8, 1):
        ark.init()
        ark.set_rank(0)
        ark.set_world_size(world)
        x, rope = ark.tensor([2048, 4096], ark.fp16), ark.tensor([1, 2048, 1, 128], ark.fp16)
        w = layer_weights(cfg, ark.fp16, world)
        decoder_layer(x, w, cfg, 1, 2048, 0, world, rope=rope, causal=True)
        lines = ark.plan_dump(str(ark.Planner(0, num_sm=148).plan())).splitlines()
        first = next(i for i, l in enumerate(lines) if " Matmul " in l)
        if world == 8:
            assert [l.split()[1] for l in lines[first:first + 3]] == ["[0,49)", "[49,98)", "[98,147)"], lines[first:first + 3]
            assert all("N=512" in l and "units=48" in l for l in lines[first:first + 3])
            assert "sync group" in lines[first - 1] and "sync group" in lines[first + 3] and "PrefillAttention" in lines[first + 4]
        else:
            assert all(l.split()[1] == "[0,148)" for l in lines[first:first + 3])
    # fewer K/V heads than query heads (70B shape at degree 8): Wq keeps the grid, Wk and Wv take a half each
    cfg = LlamaConfig(dim=8192, n_heads=64, n_kv_heads=8, ffn_dim=28672)
    ark.init()
    ark.set_rank(0)
    ark.set_world_size(8)
    x, rope = ark.tensor([4096, 8192], ark.bf16), ark.tensor([1, 1024, 1, 128], ark.bf16)
    decoder_layer(x, layer_weights(cfg, ark.bf16, 8), cfg, 4, 1024, 0, 8, rope=rope, causal=True)
    lines = ark.plan_dump(str(ark.Planner(0, num_sm=148).plan())).splitlines()
    first = next(i for i, l in enumerate(lines) if " Matmul " in l)
    assert [l.split()[1] for l in lines[first:first + 3]] == ["[0,148)", "[0,74)", "[74,148)"], lines[first:first + 3]
    ark.init()


def test_tensor_parallel_decode_layer_folds_the_one_shot_all_reduces():
    """With several ranks the small all_reduces of a decode layer take their input straight from the weight-streaming
    matmul (no push stage); the sum (+ residual) of the first one is left to the two matmuls that consume it (W1 and
    W3, which run as one stage over both matrices: it adds the staging slots up while it stages its activations); the
    last one of the plan, which nothing of the plan consumes, keeps its sum stage."""
    from ark_b200.llama import LlamaConfig, decoder_layer, layer_weights
    cfg = LlamaConfig(dim=4096, n_heads=32, n_kv_heads=32, ffn_dim=11008)
    ark.init()
    ark.set_rank(1)
    ark.set_world_size(8)
    x, rope = ark.tensor([1, 4096], ark.fp16), ark.tensor([1, 1, 1, 128], ark.fp16)
    w = layer_weights(cfg, ark.fp16, 8)
    kc, vc = ark.tensor([1, 4, 2048, 128], ark.fp16), ark.tensor([1, 4, 2048, 128], ark.fp16)
    decoder_layer(x, w, cfg, 1, 1, 1, 8, rope=rope, k_cache=kc, v_cache=vc)
    text = ark.plan_dump(str(ark.Planner(0, num_sm=148).plan()))
    ark.set_rank(0)
    ark.set_world_size(1)
    assert text.count("->all_reduce slots") == 2 and text.count("one-shot reduce +residual") == 1
    assert text.count("<-all_reduce sum +residual <-rmsnorm") == 1 and text.count("sum left to the consumers") == 1
    assert "one-shot push" not in text and " Add " not in text and text.count("peer barrier") == 2
    lines = text.splitlines()
    w1 = next(l for l in lines if "<-all_reduce sum" in l)
    assert "(second matrix, act=0" in w1 and len(lines) == 13, text


def test_unfolded_one_shot_push_waits_for_the_split_k_sum():
    """A weight-streaming matmul whose K is cut into ranges cannot store into the all_reduce slots itself: the sum
    stage writes the result and the push stage, which splits the tensor differently over the CTAs, follows a barrier."""
    ark.init()
    ark.set_rank(0)
    ark.set_world_size(2)
    x, w = ark.tensor([1, 8192], ark.fp16), ark.tensor([8192, 1024], ark.fp16)  # W:[K,N], K is split
    with ark.PlannerContext(sync=False):
        y = ark.matmul(x, w)
        y = ark.all_reduce(y, 0, 2, output=y)
    lines = ark.plan_dump(str(ark.Planner(0, num_sm=148).plan())).splitlines()
    ark.set_world_size(1)
    idx = {k: next(i for i, l in enumerate(lines) if k in l) for k in ("split-K sum", "one-shot push")}
    assert idx["one-shot push"] == idx["split-K sum"] + 2 and "sync group" in lines[idx["split-K sum"] + 1]
    assert "->all_reduce slots" not in "\n".join(lines)


def test_naive_all_reduce_composition_matches_reference_structure():
    """Model::all_reduce of the reference: world_size-1 rounds of send/send_done/recv/add (ops_all_reduce.cpp:8-37)."""
    ark.init()
    ark.set_rank(0)
    ark.set_world_size(4)
    t = ark.tensor([1024], ark.fp16)
    ark.all_reduce(t, 0, 4, naive=True)
    types = [o.type for o in ark.Model.get_model().ops if not o.virtual]
    assert types == ["Copy"] + ["Send", "SendDone", "Recv", "Add"] * 3
    ark.set_world_size(1)


from tests.conftest import reference_dir  # noqa: E402


@pytest.mark.skipif(reference_dir() is None, reason="reference checkout not present")
def test_reference_tutorial_plans_load_unmodified():
    """Plan files written for the reference (CUDA_80, 108 processors) lower as they are."""
    n = 0
    for f in sorted(glob.glob(os.path.join(reference_dir(), "examples", "tutorial", "**", "*.json"), recursive=True)):
        s = open(f).read()
        if '"TaskInfos"' not in s:
            continue
        stages, arena, procs = ark.plan_check(s)
        assert stages > 0 and procs == json.loads(s)["NumProcessors"]
        n += 1
    assert n >= 20  # 4 single-GPU tutorial plans + the two 8-rank all_reduce plan sets


def test_arena_lifetime_planner_shares_only_dead_intermediates():
    """"ArenaReuse": buffers some op writes before any op reads them, with whole-buffer dense tensors and no tags,
    may share space when their lifetimes (in processor groups, with a step of slack) do not overlap. Inputs,
    outputs and everything else keep their own space, and the default keeps the reference's layout."""
    def build(n):
        ark.init()
        x = ark.tensor([256, 1024], ark.fp16)
        t = x
        for _ in range(n):
            t = ark.relu(ark.add(t, 1.0))
        return x, t
    x, y = build(8)
    plain = ark.Planner(0, num_sm=148).plan()
    reuse = ark.Planner(0, num_sm=148, reuse_memory=True).plan()
    assert "ArenaReuse" not in plain.plan and reuse.plan["ArenaReuse"] is True
    _, a_plain, _ = ark.plan_check(str(plain))
    _, a_reuse, _ = ark.plan_check(str(reuse))
    one = 256 * 1024 * 2
    assert a_plain == 17 * one          # x + 16 results, bump-allocated as in the reference
    # x (input) and y (output, never read) keep their space; the 15 intermediates cycle through 3 blocks
    # (alive [k, k+1], one step of slack on either side)
    assert a_reuse == 5 * one, a_reuse // one
    # a buffer with a tag or a sharded view is never shared
    ark.init()
    ark.set_rank(0)
    ark.set_world_size(2)
    t = ark.relu(ark.add(ark.tensor([4096], ark.fp16), 1.0))
    t = ark.all_reduce(t, 0, 2, output=t)
    ark.relu(ark.add(t, 1.0))
    text = ark.plan_dump(str(ark.Planner(0, num_sm=148, reuse_memory=True).plan()))
    ark.set_world_size(1)
    assert "arena=" in text


def ref_allreduce_plans():
    import gzip
    with gzip.open(os.path.join(ROOT, "tests", "golden", "ref_allreduce_plans.json.gz"), "rt") as f:
        return json.load(f)


def test_reference_all_reduce_plan_sets_lower_unmodified():
    """The two 8-rank plan sets the reference ships (written for ROCM_942: 56 and 8 processors, LL8 packets) lower as
    they are: plain-data shards + DeviceSync + RecvReduceSend, and SendPacket / RecvReduceSendPacket / RecvPacket."""
    plans = ref_allreduce_plans()
    assert len(plans) == 16
    for name, text in plans.items():
        stages, arena, procs = ark.plan_check(text)
        dump = ark.plan_dump(text)
        if name.startswith("allreduce-sm"):
            assert procs == 56 and dump.count(" Send ") == 7 and "RecvReduceSend recv_reduce_send peers=7" in dump
            assert "peer barrier #1 (DeviceSync" in dump
        else:
            assert procs == 8 and dump.count(") SendPacket") == 7 and dump.count(") RecvPacket") == 7
            assert "RecvReduceSendPacket recv_reduce_send_packet peers=7 bytes=2048 packets" in dump
            assert "sync group" not in dump  # senders, reducer and receivers run side by side on their own processors


def test_packet_and_plain_all_reduce_compositions_plan_like_the_reference():
    """ark.all_reduce_packet / ark.all_reduce_sm build the op sequences of ops_all_reduce_test.cpp:52-187."""
    ark.init()
    ark.set_rank(2)
    ark.set_world_size(4)
    t = ark.tensor([8192], ark.fp16)
    ark.all_reduce_packet(t, 2, 4, 1, t)
    types = [o.type for o in ark.Model.get_model().ops if not o.virtual]
    assert types == ["SendPacket"] * 3 + ["RecvReduceSendPacket"] + ["RecvPacket"] * 3
    ops = [o for o in ark.Model.get_model().ops if not o.virtual]
    # flag 1: second half of the double-buffered scratch; rank 2 lands in slot 1 of ranks 0 and 1, slot 2 of rank 3
    nb = 8192 // 4 * 2
    assert [o.writes[0].offsets[0] for o in ops[:3]] == [nb * 3 * 2 + nb * 2 * 1, nb * 3 * 2 + nb * 2 * 1, nb * 3 * 2 + nb * 2 * 2]
    assert ops[3].reads[1].shape == [nb * 2 * 3] and ops[3].reads[1].buffer.recv_tags == [[0, ops[3].reads[1].buffer.recv_tags[0][1]], [1, ops[3].reads[1].buffer.recv_tags[0][1]], [3, ops[3].reads[1].buffer.recv_tags[0][1]]]
    ark.plan_check(str(ark.Planner(0, num_sm=148).plan()))
    ark.init()
    ark.set_rank(2)
    ark.set_world_size(4)
    t = ark.tensor([65536], ark.fp16)
    ark.all_reduce_sm(t, 2, 4)
    types = [o.type for o in ark.Model.get_model().ops if not o.virtual]
    assert types == ["Send"] * 3 + ["DeviceSync", "RecvReduceSend"] + ["Recv"] * 3 + ["DeviceSync"]
    dump = ark.plan_dump(str(ark.Planner(0, num_sm=148).plan()))
    assert dump.count("peer barrier") == 2 and "signal" not in dump
    ark.set_rank(0)
    ark.set_world_size(1)


_GLOO_WORKER = r"""
import os, sys, ctypes
import numpy as np
import torch.distributed as dist
sys.path.insert(0, sys.argv[1])
from ark_b200.executor import torch_allgather
dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{sys.argv[2]}", rank=int(sys.argv[3]), world_size=2)
rank = dist.get_rank()
fn = torch_allgather()
send = (ctypes.c_uint8 * 64)(*[(rank * 100 + i) % 256 for i in range(64)])
recv = (ctypes.c_uint8 * 128)()
rc = fn(None, ctypes.addressof(send), ctypes.addressof(recv), 64)
got = np.frombuffer(recv, dtype=np.uint8)
want = np.concatenate([np.array([(r * 100 + i) % 256 for i in range(64)], dtype=np.uint8) for r in range(2)])
assert rc == 0 and np.array_equal(got, want), (rc, got[:8])
# rank-specific shards of the benchmark operands: disjoint column / row blocks of the same matrices
import ark_b200 as ark
ark.init(); ark.set_rank(rank); ark.set_world_size(2)
from ark_b200.ffn import build_ffn
x, w1, w2, y = build_ffn(256, 512, 2048, ark.fp16, rank, 2)
assert w1.shape == [512, 1024] and w2.shape == [1024, 512]
stages, arena, procs = ark.plan_check(str(ark.Planner(0, num_sm=148).plan()))
assert stages > 3
dist.barrier(); dist.destroy_process_group()
print("ok", rank)
"""


def test_bootstrap_allgather_over_gloo_world_size_2(tmp_path):
    script = tmp_path / "w.py"
    script.write_text(_GLOO_WORKER)
    port = 29500 + (os.getpid() % 2000)
    procs = [subprocess.Popen([sys.executable, str(script), ROOT, str(port), str(r)], stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = [p.communicate(timeout=240)[0] for p in procs]
    for p, o in zip(procs, outs):
        assert p.returncode == 0, o
