"""The balance planner on the CPU: invariants of the plan for random and skewed routings."""
import pytest
import torch


def _all_topk(r, s, k, e, seed, skew):
    g = torch.Generator().manual_seed(seed)
    if skew:
        p = torch.ones(e)
        p[: max(1, e // 8)] = 12.0          # a few hot experts on the first ranks
        return torch.stack([torch.multinomial(p, s * k, replacement=True, generator=g) for _ in range(r)]).to(torch.int32)
    return torch.randint(0, e, (r, s * k), generator=g, dtype=torch.int32)


@pytest.mark.parametrize("r,s,k,e,b,pad,skew", [
    (2, 2, 1, 2, 1, 1, False), (4, 64, 4, 32, 8, 1, False), (4, 64, 4, 32, 8, 16, True), (8, 128, 8, 64, 4, 8, True),
    (8, 32, 2, 16, 2, 128, True), (1, 16, 2, 4, 2, 4, False),
])
def test_reference_plan_invariants(r, s, k, e, b, pad, skew):
    import tilexr_b200 as txr

    topk = _all_topk(r, s, k, e, 7, skew)
    n, per = s * k, e // r
    plans = [txr._C.moonep_reference_plan(topk, rank, s, k, e, b, pad) for rank in range(r)]
    nvs = plans[0]["NvS"]
    assert nvs == n + (pad - 1) * 2 * per
    # every rank computes the same slot assignment
    for p in plans[1:]:
        assert torch.equal(p["experts_to_copy"], plans[0]["experts_to_copy"])
    taken = [set() for _ in range(r)]
    received = [0] * r
    for rank in range(r):
        dst = plans[rank]["dst"]
        assert (dst >= 0).all()
        for i, raw in enumerate(dst.tolist()):
            d, slot = divmod(raw, nvs)
            assert d < r and slot not in taken[d]
            taken[d].add(slot)
            received[d] += 1
            # the slot lies inside the group of the route's expert at that destination
            expert = int(topk[rank, i])
            cu = plans[d]["cu_seqlens"].tolist()
            etc = plans[d]["experts_to_copy"][d].tolist()
            group = e + etc.index(expert) if expert in etc else expert
            begin = 0 if group == 0 else cu[group - 1]
            assert begin <= slot < cu[group]
            if group < e and not (d * per <= expert < (d + 1) * per):
                pytest.fail("a remote expert without a prefetch slot received rows")
    # balanced: every rank receives exactly N rows unless slots ran out
    assert sum(received) == r * n
    if b == per:
        assert all(x == n for x in received)
    for rank in range(r):
        cu = plans[rank]["cu_seqlens"].tolist()
        assert all(x <= y for x, y in zip(cu, cu[1:])) and cu[-1] <= nvs
        assert all(c % pad == 0 for c in cu)
        zf = plans[rank]["zero_fill_ranges"]
        padded = sum(int(x) for x in zf[:, 1])
        assert padded == nvs - received[rank]


def test_capabilities():
    import tilexr_b200 as txr

    abi, native, stub = txr._C.moonep_capabilities()
    assert abi == 2 and native == 0b11111 and stub == 0


def test_context_and_capability_objects(monkeypatch):
    """The context validates its shape like the reference's (integrations/moonep_torch/tilexr_moonep/torch_api.py:306-443),
    reads the launcher's environment, belongs to one buffer at a time and stays refused once poisoned."""
    import torch
    from tilexr_b200.integrations import moonep

    caps = moonep.NativeCapabilities.query()
    assert caps.abi_version == 2 and caps.transport_correctness_valid and not caps.transport_performance_valid
    assert all(caps.implementation(s) == "native" for s in moonep.STAGE_BITS)
    assert moonep.NativeCapabilities(2, 0b00111, 0b00100).implementation("prefetch_weight") == "stub"
    assert moonep.NativeCapabilities(2, 0b00111, 0).implementation("combine") == "unavailable"
    with pytest.raises(KeyError):
        caps.implementation("scatter")

    class FakeComm:
        rank, world_size = 3, 8

    for key, value in {"RANK": "3", "WORLD_SIZE": "8", "LOCAL_RANK": "0", "LOCAL_WORLD_SIZE": "8", "NODE_RANK": "0", "NODE_COUNT": "1"}.items():
        monkeypatch.setenv(key, value)
    monkeypatch.setattr(torch.cuda, "is_available", lambda: False)
    ctx = moonep.TileXRMoonEPContext.from_env(tokens_per_rank=4096, hidden_size=7168, topk=8, expert_count=256, dtype=torch.bfloat16,
                                              token_padding=16, runtime=FakeComm())
    assert (ctx.planner_group_rank, ctx.planner_group_size, ctx.experts_per_rank, ctx.prefetch_slots) == (3, 8, 32, 32)
    assert ctx.route_count == 32768 and ctx.nv_s == 32768 + 15 * 2 * 32 and ctx.dispatched_capacity == ctx.nv_s
    a, b = object(), object()
    ctx.attach_buffer(a)
    with pytest.raises(RuntimeError):
        ctx.attach_buffer(b)
    ctx.bind_stream(a, 7)
    with pytest.raises(RuntimeError):
        ctx.bind_stream(a, 9)
    with pytest.raises(RuntimeError):
        ctx.close()                       # its buffer first
    ctx.detach_buffer(a)
    ctx.mark_poisoned()
    with pytest.raises(RuntimeError):
        ctx.attach_buffer(b)
    ctx.close()

    def make(**kw):
        base = dict(runtime=FakeComm(), global_rank=3, global_world_size=8, node_rank=0, node_count=1, local_rank=3, local_world_size=8,
                    planner_group_rank=3, planner_group_size=8, lane_group_rank=0, lane_group_size=1, device_index=3, tokens_per_rank=64,
                    hidden_size=128, topk=4, expert_count=32, dtype=torch.bfloat16)
        base.update(kw)
        return moonep.TileXRMoonEPContext(**base)

    assert make().prefetch_slots == 4
    for bad in (dict(topk=33), dict(expert_count=30), dict(prefetch_slots=5), dict(token_padding=0), dict(planner_group_rank=8),
                dict(planner_group_rank=2), dict(tokens_per_rank=1 << 28, topk=8)):
        with pytest.raises((ValueError, OverflowError)):
            make(**bad)


def test_stage_tracing_and_latency_capture_from_the_environment(monkeypatch, tmp_path, capsys):
    """TILEXR_MOONEP_TRACE_STAGES / TILEXR_MOONEP_PERF_CAPTURE_* on a buffer whose native calls are replaced by no-ops: the stage
    names of a forward and a backward pass in call order, skipped warm-up calls, the per-rank file and its merge into one
    document (reference: integrations/moonep_torch/tilexr_moonep/torch_api.py:669-790)."""
    import json

    import torch
    from tilexr_b200.integrations import moonep, moonep_capture
    from tilexr_b200.tools.moonep import model_flow

    class FakeComm:
        rank, world_size = 1, 2

        def symm_empty(self, shape, dtype):
            return torch.zeros(shape, dtype=dtype)

    plan_dict = {"dst": torch.zeros(8, dtype=torch.int32), "experts_to_copy": torch.zeros(2, 2, dtype=torch.int32), "zero_fill_ranges": torch.zeros(6, 2, dtype=torch.int32),
                 "remote_stats": torch.zeros(2, dtype=torch.int32), "N": 8, "R": 2, "E": 4, "B": 2, "NvS": 8, "K": 2, "dup_counts": None, "status": None,
                 "dst_local": None, "cu_seqlens": torch.zeros(6, dtype=torch.int32)}
    monkeypatch.setattr(moonep._C, "moonep_planning", lambda *a, **k: dict(plan_dict), raising=False)
    for name in ("moonep_dispatch", "moonep_prefetch_weight", "moonep_combine", "moonep_reduce_grad"):
        monkeypatch.setattr(moonep._C, name, lambda *a, **k: None, raising=False)
    monkeypatch.setattr(torch.cuda, "is_available", lambda: False)
    monkeypatch.setenv("TILEXR_MOONEP_TRACE_STAGES", "1")
    monkeypatch.setenv("TILEXR_MOONEP_PERF_CAPTURE_DIR", str(tmp_path))
    monkeypatch.setenv("TILEXR_MOONEP_PERF_CAPTURE_ID", "unit")
    monkeypatch.setenv("TILEXR_MOONEP_PERF_CAPTURE_OPERATORS", "7")
    monkeypatch.setenv("TILEXR_MOONEP_PERF_CAPTURE_SKIP_OPERATORS", "4")
    buf = moonep.TileXRMoonEPBuffer(FakeComm(), S=4, H=8, K=2, E=4, token_padding=1, dtype=torch.float32)
    hidden, w, topk = torch.zeros(4, 8), torch.ones(4, 2), torch.zeros(4, 2, dtype=torch.int32)
    proj = moonep.ProjectionBuffers(torch.zeros(4, 2, 8), torch.zeros(4, 2, 8), torch.zeros(4, 2, 8))
    for _ in range(2):                                            # the first forward (4 calls) is the skipped warm-up
        y, plan = buf.forward(hidden, w, topk, None, proj, lambda rows, cu, p: rows)
    buf.backward(hidden, plan, lambda rows, cu: rows, grads=proj)
    buf.close()
    traced = [line for line in capsys.readouterr().err.splitlines() if "TileXR MoonEP rank 1" in line]
    assert len(traced) == 11 and "planning (call 0)" in traced[0] and "reduce_grad (call 10)" in traced[-1]
    doc = json.loads((tmp_path / "rank1_performance.json").read_text())
    assert doc["capture_id"] == "unit" and doc["complete"] and doc["rank"] == 1
    assert [o["stage"] for o in doc["operators"]] == ["planning", "dispatch_forward", "prefetch_weight", "combine_forward", "dispatch_backward",
                                                      "combine_backward", "reduce_grad"]
    assert [o["source_operator"] for o in doc["operators"]] == list(range(4, 11)) and all(o["latency_us"] >= 0 for o in doc["operators"])
    merged = moonep_capture.merge_capture_files(str(tmp_path))
    assert set(model_flow.stage_medians(merged)) == set(model_flow.FORWARD_STAGES + model_flow.BACKWARD_STAGES)
    # a directory without an id is refused when the buffer is made
    monkeypatch.delenv("TILEXR_MOONEP_PERF_CAPTURE_ID")
    with pytest.raises(ValueError):
        moonep.TileXRMoonEPBuffer(FakeComm(), S=4, H=8, K=2, E=4, token_padding=1, dtype=torch.float32)
    # off by default: nothing is timed, nothing is written
    for name in ("TILEXR_MOONEP_TRACE_STAGES", "TILEXR_MOONEP_PERF_CAPTURE_DIR"):
        monkeypatch.delenv(name)
    quiet = moonep.TileXRMoonEPBuffer(FakeComm(), S=4, H=8, K=2, E=4, token_padding=1, dtype=torch.float32)
    assert not quiet._capture.active
    quiet.forward(hidden, w, topk, None, None, lambda rows, cu, p: rows)
    assert quiet._capture.seen == 0


def test_drop_in_buffer_accepts_the_zero_copy_and_sync_switches(monkeypatch):
    """`zero_copy` / `inter_rank_sync` of the drop-in Buffer (reference: integrations/moonep_torch/tilexr_moonep/compat.py:264-330,
    407-458): accepted; a zero-copy combine wants exactly the tensors of the latest zero-copy dispatch of the same plan."""
    import torch
    from tilexr_b200.integrations import moonep

    class FakeComm:
        rank, world_size = 0, 1

        def symm_empty(self, shape, dtype):
            return torch.zeros(shape, dtype=dtype)

    plan_dict = {"dst": torch.zeros(8, dtype=torch.int32), "experts_to_copy": torch.zeros(1, 4, dtype=torch.int32), "zero_fill_ranges": torch.zeros(8, 2, dtype=torch.int32),
                 "remote_stats": torch.zeros(2, dtype=torch.int32), "N": 8, "R": 1, "E": 4, "B": 4, "NvS": 8, "K": 2, "dup_counts": None, "status": None,
                 "dst_local": None, "cu_seqlens": torch.zeros(8, dtype=torch.int32)}
    monkeypatch.setattr(moonep._C, "moonep_planning", lambda *a, **k: dict(plan_dict), raising=False)
    for name in ("moonep_dispatch", "moonep_combine"):
        monkeypatch.setattr(moonep._C, name, lambda *a, **k: None, raising=False)
    monkeypatch.setattr(torch.cuda, "is_available", lambda: False)
    buf = moonep.Buffer(4, 8, 2, 4, 1, token_padding=1, comm=FakeComm(), dtype=torch.float32)
    hidden, w, topk = torch.zeros(4, 8), torch.ones(4, 2), torch.zeros(4, 2, dtype=torch.int32)
    rows, wn, cu, plan = buf.dispatch(hidden, w, topk, zero_copy=True, inter_rank_sync=False)
    y, wk, ev = buf.combine(plan, rows, wn, zero_copy=True, inter_rank_sync=False)
    assert y.shape == (4, 8) and ev is None
    with pytest.raises(AssertionError):
        buf.combine(plan, rows, wn, zero_copy=True)               # the aliases are used up
    rows, wn, cu, plan = buf.dispatch(hidden, w, plan=plan, zero_copy=True)
    with pytest.raises(AssertionError):
        buf.combine(plan, rows.clone(), wn, zero_copy=True)       # another tensor
    rows, wn, cu, plan = buf.dispatch(hidden, w, plan=plan, zero_copy=True)
    with pytest.raises(AssertionError):
        buf.combine(plan.clone(), rows, wn, zero_copy=True)       # another plan
    buf.combine(plan, rows, wn)                                   # without the switch nothing is checked
    buf.destroy()
    assert buf.destroyed


def test_plan_file_round_trip_and_checks(tmp_path):
    """A plan saved after planning dispatches again later without planning: every table survives the file, a plan made for
    another shape or a cut table is refused."""
    import dataclasses

    from tilexr_b200.integrations.moonep import MoonEPCommPlan, TileXRMoonEPError
    from tilexr_b200.tools.moonep.case_factory import load_cases, routing
    from tilexr_b200.tools.moonep.planner_reference import dst_local_from_plans, reference_plan

    case = [c for c in load_cases("smoke") if c.ranks == 2][0]
    topk = [routing(case, r) for r in range(case.ranks)]
    raw = [reference_plan(case, topk, r) for r in range(case.ranks)]
    p = raw[0]
    plan = MoonEPCommPlan(p["dst"].to(torch.int32), p["experts_to_copy"].to(torch.int32), p["zero_fill_ranges"], p["remote_stats"], case.routes, case.ranks,
                          case.experts, case.prefetch_slots, case.nvs, case.top_k, dup_groups=torch.arange(6, dtype=torch.int32),
                          dup_loffs=torch.arange(3, dtype=torch.int32), dup_counts=torch.tensor([3], dtype=torch.int32),
                          status=torch.zeros(4, dtype=torch.int32), dst_local=dst_local_from_plans(case, [x["dst"] for x in raw], 0).to(torch.int32),
                          cu_seqlens=p.get("cu_seqlens"))
    path = str(tmp_path / "plan.pt")
    plan.save(path)
    shape = {"N": case.routes, "R": case.ranks, "E": case.experts, "B": case.prefetch_slots, "NvS": case.nvs, "K": case.top_k}
    back = MoonEPCommPlan.load(path, expect=shape)
    for f in dataclasses.fields(MoonEPCommPlan):
        a, b = getattr(plan, f.name), getattr(back, f.name)
        assert (a is None and b is None) or (torch.equal(a, b) and a.dtype == b.dtype) if isinstance(a, torch.Tensor) or a is None else a == b, f.name
    assert MoonEPCommPlan.load(path, device="cpu").dst.device.type == "cpu"
    with pytest.raises(TileXRMoonEPError, match="K = 2"):
        MoonEPCommPlan.load(path, expect=dict(shape, K=4))
    cut = plan.clone()
    cut.dst = cut.dst[:-1]
    cut.save(path)
    with pytest.raises(TileXRMoonEPError, match="table dst"):
        MoonEPCommPlan.load(path)
    torch.save({"version": 99}, path)
    with pytest.raises(TileXRMoonEPError, match="version"):
        MoonEPCommPlan.load(path)
