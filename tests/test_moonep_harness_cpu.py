"""MoonEP harness on the CPU: the torch reference backend over gloo, the correctness runner's verdicts, plan
invariants, the HMAC completion barrier and the route capture format."""
import dataclasses
import os
import threading

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import free_port


def _gloo_worker(rank, world, port, q):
    try:
        dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
        from tilexr_b200.tools.moonep.case_factory import load_cases
        from tilexr_b200.tools.moonep.correctness import CorrectnessRunner
        from tilexr_b200.tools.moonep.torch_reference_backend import TorchReferenceBackend

        case = [c for c in load_cases("smoke") if c.ranks == world][0]
        ref = TorchReferenceBackend()

        class Faulty(TorchReferenceBackend):
            name = "faulty"

            def run(self, case, inputs, expert_rows=None):
                art = super().run(case, inputs)
                if dist.get_rank() == 1:
                    art.combined_hidden[3, 5] += 1.0          # one wrong element on one rank
                return art

        class Scribbler(TorchReferenceBackend):
            name = "scribbler"

            def run(self, case, inputs, expert_rows=None):
                art = super().run(case, inputs)
                inputs.hidden_sh[0, 0] += 1.0                 # a backend must not touch its inputs
                return art

        good = CorrectnessRunner(ref, TorchReferenceBackend()).run_case(case)
        bad = CorrectnessRunner(ref, Faulty()).run_case(case)
        scribble = CorrectnessRunner(ref, Scribbler()).run_case(case)
        q.put((rank, good, bad, scribble))
        dist.destroy_process_group()
    except Exception:
        import traceback

        q.put((rank, traceback.format_exc(), None, None))


def test_reference_backend_and_runner_verdicts_over_gloo():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=_gloo_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = sorted((q.get(timeout=180) for _ in procs), key=lambda r: r[0])
    for p in procs:
        p.join(timeout=30)
    for rank, good, bad, scribble in results:
        assert isinstance(good, dict), good
        assert good["ok"] and good["ok_all_ranks"]
        assert not bad["ok_all_ranks"]                          # every rank learns that the case failed
        failing = [s["stage"] for s in bad["stages"] if not s["ok"]]
        assert failing == (["combined_hidden"] if rank == 1 else [])
        assert [s["stage"] for s in scribble["stages"] if not s["ok"]] == ["inputs_immutable"]


def _host_backend_worker(rank, world, port, q):
    try:
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        dist.init_process_group("gloo", rank=rank, world_size=world)
        import tilexr_b200 as txr
        from tilexr_b200.tools.moonep.case_factory import load_cases, make_inputs
        from tilexr_b200.tools.moonep.correctness import CorrectnessRunner
        from tilexr_b200.tools.moonep.host_backend import HostMemoryBackend
        from tilexr_b200.tools.moonep.torch_reference_backend import TorchReferenceBackend

        comm = txr.init_from_torch_distributed(host_memory=True, buffer_mb=32)
        case = [c for c in load_cases("smoke") if c.ranks == world][0]
        backend = HostMemoryBackend(comm)
        runner = CorrectnessRunner(TorchReferenceBackend(), backend)
        first = runner.run_case(case)
        again = runner.run_case(dataclasses.replace(case, seed=case.seed + 5))      # other routing, same windows: both halves, the reuse guard
        padded = runner.run_case(dataclasses.replace(case, token_padding=4, seed=9))
        # an expert function between dispatch and combine: the sum is of what the experts returned
        inputs = make_inputs(case, rank)
        art = backend.run(case, inputs, expert_fn=lambda rows, plan: rows * 2)
        doubled = torch.equal(art.combined_hidden.float(), (backend.run(case, inputs).combined_hidden.float() * 2))
        # a rank that raises no flag: the others' dispatch ends with a status instead of waiting for ever
        status = None
        if world > 1:
            comm.set_wait_timeout_ms(300)
            dist.barrier()
            if rank == 0:
                # one launch without flags and nothing after it (flags are compared with >=: a later launch's flags would
                # release the waiting ranks)
                txr._C.host_inject_skip_flags(True)
                backend._all_gather(inputs.topk_experts_sk.to(torch.int32))
                status = "withheld"
            else:
                try:
                    backend.run(case, inputs)
                    status = "finished"
                except RuntimeError as e:
                    status = str(e)
        q.put((rank, first, again, padded, doubled, status))
        dist.destroy_process_group()
    except Exception:
        import traceback

        q.put((rank, traceback.format_exc(), None, None, None, None))


@pytest.mark.parametrize("world", [2, 4])
def test_host_memory_backend_matches_the_reference_backend(world):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=_host_backend_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = sorted((q.get(timeout=240) for _ in procs), key=lambda r: r[0])
    for p in procs:
        p.join(timeout=30)
    for rank, first, again, padded, doubled, status in results:
        assert isinstance(first, dict), first
        for verdict in (first, again, padded):
            assert verdict["ok_all_ranks"], [s for s in verdict["stages"] if not s["ok"]]
        assert doubled
    # every rank but the one that withheld its flags reports the wait that ran out
    assert results[0][5] == "withheld"
    assert all("timeout" in r[5] for r in results[1:]), [r[5] for r in results]


def test_plan_invariants_hold_for_reference_plans_and_catch_a_collision():
    from tilexr_b200.tools.moonep.case_factory import load_cases, routing
    from tilexr_b200.tools.moonep.planner_reference import check_plan_invariants, dst_local_from_plans, reference_plan

    for case in load_cases("correctness"):
        topk = [routing(case, r) for r in range(case.ranks)]
        plans = [reference_plan(case, topk, r) for r in range(case.ranks)]
        assert check_plan_invariants(case, plans) == [], case.name
        for r in range(case.ranks):
            dl = dst_local_from_plans(case, [p["dst"] for p in plans], r)
            assert int((dl >= 0).sum()) <= case.nvs
        total = sum(int((dst_local_from_plans(case, [p["dst"] for p in plans], r) >= 0).sum()) for r in range(case.ranks))
        assert total == case.ranks * case.routes               # every route lands exactly once
    case = load_cases("smoke")[0]
    topk = [routing(case, r) for r in range(case.ranks)]
    plans = [reference_plan(case, topk, r) for r in range(case.ranks)]
    plans[1]["dst"] = plans[1]["dst"].clone()
    plans[1]["dst"][1] = plans[1]["dst"][0]                     # two routes into one slot
    assert any("used twice" in v for v in check_plan_invariants(case, plans))


def test_plan_invariants_hold_for_v2_plans():
    """The topology-aware planner's oracle through the harness: the same invariants, with duplicate routes encoded."""
    from tilexr_b200.tools.moonep.case_factory import load_cases, routing
    from tilexr_b200.tools.moonep.planner_reference import check_plan_invariants, reference_plan_v2

    checked = 0
    for case in load_cases("correctness"):
        topk = [routing(case, r) for r in range(case.ranks)]
        plans = [reference_plan_v2(case, topk, r, nvs=case.ranks * case.routes) for r in range(case.ranks)]
        assert all(int(p["code"]) <= 3 for p in plans), (case.name, [p["status"].tolist() for p in plans])
        assert check_plan_invariants(case, plans) == [], case.name
        codes = {int(p["code"]) for p in plans}
        assert len(codes) == 1                                   # every rank reaches the same verdict
        if codes == {0}:
            per_rank = [0] * case.ranks
            for p in plans:
                raw = torch.where(p["dst"] >= 0, p["dst"], ~p["dst"]).to(torch.int64)
                for r in range(case.ranks):
                    per_rank[r] += int((raw // p["NvS"] == r).sum())
            assert per_rank == [case.routes] * case.ranks, (case.name, per_rank)     # balanced to the capacity
        checked += 1
    assert checked > 0


def test_ulp_distance_and_compare_policies():
    from tilexr_b200.tools.moonep.correctness import compare, ulp_distance

    a = torch.tensor([1.0, -2.0, 0.5], dtype=torch.bfloat16)
    b = a.clone()
    assert ulp_distance(a, b) == 0
    b[0] = torch.nextafter(a[0].float(), torch.tensor(2.0)).to(torch.bfloat16) if False else torch.tensor(1.0078125, dtype=torch.bfloat16)
    assert ulp_distance(a, b) == 1
    assert compare("combined_hidden", a, b).ok                  # one ulp is within the policy
    assert not compare("dispatched_hidden", a, b).ok            # copies must be bit-exact
    b[0] = torch.tensor(1.015625, dtype=torch.bfloat16)
    assert not compare("combined_hidden", a, b).ok
    assert compare("prefetched_gate", None, None).ok and not compare("prefetched_gate", a, None).ok


def test_completion_barrier_ignores_unauthenticated_frames():
    import socket

    from tilexr_b200.tools.moonep.rendezvous import completion_barrier

    port = free_port()
    world = 3
    out = [None] * world

    def run(rank):
        out[rank] = completion_barrier(rank, world, "127.0.0.1", port, b"secret", "t1", timeout_s=20)

    threads = [threading.Thread(target=run, args=(r,)) for r in range(world)]
    threads[0].start()
    # a stranger with the wrong key talks to the server first
    for _ in range(100):
        try:
            with socket.create_connection(("127.0.0.1", port), timeout=0.2) as s:
                s.sendall(b"\\x00\\x00\\x00\\x02{}" + b"0" * 32)
            break
        except OSError:
            import time

            time.sleep(0.05)
    for t in threads[1:]:
        t.start()
    for t in threads:
        t.join(timeout=30)
    assert out == [True, True, True]
    assert completion_barrier(1, 2, "127.0.0.1", free_port(), b"k", "nobody-listens", timeout_s=0.5) is False


def test_route_capture_round_trip_and_compare(tmp_path):
    from tilexr_b200.tools.moonep.model_replay import RouteRecorder, compare_replays, layer_case, load_meta

    for rank in range(2):
        rec = RouteRecorder(str(tmp_path), rank, ranks=2, experts=8, prefetch_slots=2, token_padding=4)
        for layer in range(3):
            rec.record(f"layers.{layer}.moe", torch.randint(0, 8, (16, 2)), hidden=128)
        rec.save()
    meta = load_meta(str(tmp_path))
    assert [l["name"] for l in meta["layers"]] == ["layers.0.moe", "layers.1.moe", "layers.2.moe"]
    case = layer_case(meta, meta["layers"][1])
    assert (case.ranks, case.tokens, case.top_k, case.hidden, case.experts) == (2, 16, 2, 128, 8)
    case.validate()
    assert (tmp_path / "layer0002_rank1.pt").exists()
    rows = compare_replays({"total_us": {"dispatch_fwd": 200.0}}, {"total_us": {"dispatch_fwd": 100.0}})
    assert rows[0]["speedup_b_over_a"] == 2.0


def test_expert_forward_matches_a_per_expert_loop():
    from tilexr_b200.tools.moonep.expert_forward import expert_forward

    g = torch.Generator().manual_seed(0)
    rows = torch.randn(20, 32, generator=g)
    gate, up, down = (torch.randn(3, 16, 32, generator=g) * 0.1 for _ in range(3))
    cu = torch.tensor([5, 5, 14])                  # expert 1 got nothing; rows 14.. are padding
    out = expert_forward(rows, cu, gate, up, down)
    assert torch.all(out[14:] == 0)
    for j, (s, e) in enumerate([(0, 5), (5, 5), (5, 14)]):
        if e > s:
            want = (torch.nn.functional.silu(rows[s:e] @ gate[j].t()) * (rows[s:e] @ up[j].t())) @ down[j]
            assert torch.allclose(out[s:e], want, atol=1e-5)


def test_report_statistics_and_rank_aggregation(tmp_path):
    import math

    from tilexr_b200.tools.moonep import report

    assert report.percentile([1, 2, 3, 4], 0.5) == 2.5
    assert report.percentile([5.0], 0.99) == 5.0
    assert math.isnan(report.percentile([], 0.5))
    s = report.metric_summary([10.0, 0.5, 30.0, 20.0, 1.0])          # 0.5 and 1.0 us did not bracket a kernel
    assert s["samples"] == 5 and s["invalid"] == 2 and s["p50"] == 20.0 and s["min"] == 10.0 and s["max"] == 30.0
    assert math.isnan(report.metric_summary([0.2, 0.9])["p50"])
    agg = report.aggregate_rank_samples([[10, 20, 30], [12, 18, 33], [11, 25, 29, 99]])
    assert agg["iterations"] == 3 and agg["ranks"] == 3
    assert agg["cross_rank_max"]["p50"] == 25.0 and agg["cross_rank_max"]["max"] == 33.0     # slowest rank per iteration
    assert agg["rank_p50"][:2] == [20.0, 18.0]
    # per-rank files of a multi-node run fold into the same numbers
    for r, vals in enumerate([[10, 20, 30], [12, 18, 33]]):
        report.write_jsonl(tmp_path / f"rank{r}.jsonl",
                           report.rank_sample_rows("c", r, {"dispatch": vals}, {"dispatch": 1e6 * (r + 1)}))
    rows = report.aggregate_rank_artifacts(tmp_path)
    assert len(rows) == 1 and rows[0]["stage"] == "dispatch" and rows[0]["cross_rank_max"]["p50"] == 20.0
    assert rows[0]["bytes_per_rank"] == 2e6 and abs(rows[0]["gbps_at_p50"] - 2e6 / 20.0 / 1e3) < 1e-9
    md = report.benchmark_markdown([{"case": "c", "stage_us": {"dispatch": 20.0}, "stage_stats": {"dispatch": rows[0]},
                                     "stage_bytes": {"dispatch": 2e6}, "stage_gbps": {"dispatch": 100.0}}])
    assert "| c | dispatch | 20.0 |" in md
    report.write_stage_csv(tmp_path / "s.csv", [{"case": "c", "ranks": 2, "stage_stats": {"dispatch": rows[0]},
                                                 "stage_bytes": {"dispatch": 2e6}, "stage_gbps": {"dispatch": 100.0}}])
    assert (tmp_path / "s.csv").read_text().splitlines()[1].startswith("c,2,dispatch,20.0")


def test_algorithm_bytes_follow_the_plan():
    import types

    import torch

    from tilexr_b200.tools.moonep.benchmark import algorithm_bytes
    from tilexr_b200.tools.moonep.prefetch_weight_benchmark import synthetic_borrow_table

    plan = types.SimpleNamespace(dst=torch.tensor([0, 5, 10 + 3, -(10 + 4) - 1, 2 * 10 + 1, -1 - 7], dtype=torch.int32), NvS=10, R=3,
                                 remote_stats=torch.tensor([2, 3]))
    b = algorithm_bytes(plan, rank=0, hidden_row_bytes=100, weight_bytes=4, projection_row_bytes=1000, gradient_row_bytes=2000)
    assert b["dispatch"] == b["combine"] == 3 * 204            # routes to ranks 1, 1 (duplicate) and 2
    assert b["prefetch_weight"] == 2000 and b["reduce_grad"] == 6000
    t = synthetic_borrow_table(4, 2, 3)
    for r in range(4):
        assert all(int(e) // 2 != r and 0 <= int(e) < 8 for e in t[r])          # always a remote owner
    assert (synthetic_borrow_table(1, 2, 2) == -1).all()


def test_tensor_dump_round_trip_and_offline_compare(tmp_path):
    """Stage tensors dumped by the correctness runner (single rank, the reference backend on both sides), then compared
    offline: equal by digest, a changed element found with its index, a tolerance that accepts it, a missing rank."""
    from tilexr_b200.tools.moonep import tensor_dump
    from tilexr_b200.tools.moonep.contracts import MoonEPCase
    from tilexr_b200.tools.moonep.correctness import CorrectnessRunner
    from tilexr_b200.tools.moonep.torch_reference_backend import TorchReferenceBackend

    case = MoonEPCase(name="dump-case", ranks=1, tokens=16, hidden=32, top_k=2, experts=4, prefetch_slots=2, token_padding=4, ffn=8)
    case.validate()
    r = CorrectnessRunner(TorchReferenceBackend(), TorchReferenceBackend(), dump_dir=str(tmp_path / "run")).run_case(case)
    assert r["ok"]
    ref_dir, cand_dir = tmp_path / "run" / "reference", tmp_path / "run" / "candidate"
    names = {n for m in tensor_dump.manifests(str(ref_dir)) for n in m["tensors"]}
    assert {"plan.dst", "dispatched_hidden", "combined_hidden", "prefetched_gate", "reduced_grad", "input.hidden_sh"} <= names
    rows = tensor_dump.compare_dumps(str(cand_dir), str(ref_dir))
    shared = [x for x in rows if not x["tensor"].startswith("input.")]
    assert all(x["verdict"] == "equal" for x in shared)
    assert all(x["verdict"] == "missing" and x["only_in"] == "b" for x in rows if x["tensor"].startswith("input."))
    # one element of one tensor changed in a copy of the candidate dump
    other = tmp_path / "other"
    tensors = tensor_dump.load_rank(str(cand_dir), case.name, 0)
    from tilexr_b200.tools.moonep.contracts import StageArtifacts

    changed = tensors["combined_hidden"].clone()
    changed[3, 5] += 0.5
    art = StageArtifacts(plan={k[5:]: v for k, v in tensors.items() if k.startswith("plan.")}, dispatched_hidden=tensors["dispatched_hidden"],
                         dispatched_weights=tensors["dispatched_weights"], prefetched_gate=tensors["prefetched_gate"], combined_hidden=changed,
                         combined_weights=tensors["combined_weights"], reduced_grad=tensors["reduced_grad"])
    tensor_dump.dump_rank(str(other), case, 0, art)
    rows = tensor_dump.compare_dumps(str(cand_dir), str(other))
    diff = [x for x in rows if x["verdict"] != "equal"]
    assert len(diff) == 1 and diff[0]["tensor"] == "combined_hidden" and diff[0]["verdict"] == "differs"
    assert diff[0]["first_index"] == 3 * 32 + 5 and diff[0]["mismatched"] == 1 and abs(diff[0]["max_abs"] - 0.5) < 0.01
    assert not tensor_dump.summarize(rows)["ok"]
    assert tensor_dump.summarize(tensor_dump.compare_dumps(str(cand_dir), str(other), atol=1.0))["ok"]
    assert tensor_dump.main(["compare", str(cand_dir), str(other)]) == 1 and tensor_dump.main(["compare", str(cand_dir), str(cand_dir)]) == 0
    (other / case.name / "rank0.manifest.json").unlink()
    assert [x["verdict"] for x in tensor_dump.compare_dumps(str(cand_dir), str(other))] == ["missing"]


def test_model_flow_operator_order_routes_and_document():
    """The training step's operator sequence (reference: tools/moonep/model_flow.py:55-165): 2L forward and L backward calls
    with recomputation; routes rebuilt from a histogram; the per-operator document and its comparison table."""
    import types

    from tilexr_b200.tools.moonep import model_flow as mf
    from tilexr_b200.tools.moonep.contracts import MoonEPCase

    order = mf.operator_order(5)
    assert len(order) == 55 and [o["sequence"] for o in order] == list(range(55))
    count = lambda stage: sum(o["stage"] == stage for o in order)
    assert all(count(s) == 10 for s in mf.FORWARD_STAGES) and all(count(s) == 5 for s in mf.BACKWARD_STAGES)
    assert [o["layer"] for o in order if o["stage"] == "reduce_grad"] == [4, 3, 2, 1, 0]
    assert order[20]["phase"] == "recompute_backward" and order[20]["stage"] == "planning" and order[20]["stage_occurrence"] == 5
    assert len(mf.operator_order(3, recompute=False)) == 3 * 4 + 3 * 3

    counts = [9, 0, 7, 16, 3, 5, 8, 16]                      # 16 tokens x top-4
    routes = mf.routes_from_expert_counts(counts, 16, 4)
    assert torch.bincount(routes.reshape(-1).long(), minlength=8).tolist() == counts
    assert all(len(set(row.tolist())) == 4 for row in routes)
    for bad in ([17, 15, 16, 16], [64, 0, 0, 0], [16, 16, 16, 15]):
        with pytest.raises(ValueError):
            mf.routes_from_expert_counts(bad, 16, 4)
    with pytest.raises(ValueError):
        mf.routes_from_expert_counts([16, 16, 16, 0, 0, 16], 16, 4 + 1)

    case = MoonEPCase(name="flow", ranks=2, tokens=16, hidden=32, top_k=4, experts=8, prefetch_slots=2, ffn=8)
    log = []

    class FakeBuffer:
        weights_nvs = torch.zeros(4)

        def planning(self, topk):
            log.append("planning")
            return types.SimpleNamespace(remote_stats=torch.tensor([2, 1]))

        def dispatch(self, hidden, weights, plan):
            log.append("dispatch_forward" if weights is not None else "dispatch_backward")
            return hidden, weights

        def prefetch_weight(self, plan, proj):
            log.append("prefetch_weight")

        def combine(self, plan, rows, weights=None):
            log.append("combine_backward" if weights is not None else "combine_forward")
            return rows, None

        def reduce_grad(self, plan, grads):
            log.append("reduce_grad")

    hidden = torch.zeros(16, 32)
    flow = mf.ModelFlow(FakeBuffer(), case, [torch.zeros(16, 4, dtype=torch.int32)] * 2, hidden, torch.ones(16, 4), projections=object(), grads=object())
    runs = [flow.run_iteration() for _ in range(3)]
    assert log[:22] == [o["stage"] for o in mf.operator_order(2)] and len(log) == 3 * 22
    doc0 = mf.performance_document(case, 0, runs, projection_row_bytes=3 * 8 * 32 * 2)
    doc1 = mf.performance_document(case, 1, runs, projection_row_bytes=3 * 8 * 32 * 2)
    doc = mf.merge_rank_documents([doc0, doc1])
    ops = doc["ranks"]["1"]["operators"]
    assert len(ops) == 22 and ops[0]["algorithm_bytes"] is None                      # planning moves no payload
    assert ops[1]["algorithm_bytes"] == 64 * 32 * 2 + 64 * 4                          # rows and route weights
    assert [o for o in ops if o["stage"] == "prefetch_weight"][0]["algorithm_bytes"] == 2 * 3 * 8 * 32 * 2
    assert [o for o in ops if o["stage"] == "reduce_grad"][0]["algorithm_bytes"] == 1 * 3 * 8 * 32 * 2
    med = mf.stage_medians(doc)
    assert set(med) == set(mf.FORWARD_STAGES + mf.BACKWARD_STAGES) and med["planning"]["operators"] == 4
    rows = mf.compare_with_published(doc)
    assert {r["stage"] for r in rows} == set(med) and all(r["published_us"] and r["speedup"] > 0 for r in rows)
    assert "| reduce_grad | 2 |" in mf.markdown(doc)
    # stages without buffers are skipped, not timed
    flow2 = mf.ModelFlow(FakeBuffer(), case, [torch.zeros(16, 4, dtype=torch.int32)], hidden, torch.ones(16, 4))
    rec = flow2.run_iteration()
    assert [r["stage"] for r in rec if r["skipped"]] == ["prefetch_weight", "prefetch_weight", "reduce_grad"]
    assert "prefetch_weight" not in mf.stage_medians(mf.performance_document(case, 0, [rec]))


def test_case_selection_overrides_flowchart_and_hot_loop_helpers(tmp_path):
    from tilexr_b200.tools.moonep import dispatch_hot_loop as hl, flowcharts, tensor_dump
    from tilexr_b200.tools.moonep.case_factory import apply_overrides, load_cases, make_inputs, routing, select_cases
    from tilexr_b200.tools.moonep.contracts import MoonEPCase
    from tilexr_b200.tools.moonep.correctness import CorrectnessRunner
    from tilexr_b200.tools.moonep.planner_reference import reference_plan
    from tilexr_b200.tools.moonep.torch_reference_backend import TorchReferenceBackend

    cases = load_cases("correctness")
    assert [c.name for c in select_cases(cases, "2,uniform_r2_k1")] == [cases[1].name, "uniform_r2_k1"]
    assert select_cases(cases, "") == cases
    for bad in ("0", "999", "no_such_case"):
        with pytest.raises(ValueError):
            select_cases(cases, bad)
    c = apply_overrides(cases[0], {"tokens": 48, "hidden": None, "seed": 9})
    assert (c.tokens, c.seed, c.hidden) == (48, 9, cases[0].hidden) and "tokens=48" in c.name and apply_overrides(cases[0], {}) is cases[0]
    with pytest.raises(ValueError):
        apply_overrides(cases[0], {"ranks": 4})
    with pytest.raises(ValueError):
        apply_overrides(cases[0], {"prefetch_slots": 10 ** 6})                 # validated again

    # a chart from a dump
    case = MoonEPCase(name="chart", ranks=1, tokens=8, hidden=16, top_k=2, experts=4, prefetch_slots=2, ffn=4)
    CorrectnessRunner(TorchReferenceBackend(), TorchReferenceBackend(), dump_dir=str(tmp_path / "d")).run_case(case)
    text = flowcharts.chart_from_dump(str(tmp_path / "d" / "reference"), "chart", 0)
    assert text.startswith("flowchart TD") and all(f"  {s}[" in text for s in ("planning", "dispatch", "prefetch_weight", "combine", "reduce_grad"))
    assert "dispatched_hidden [16, 16] bfloat16" in text and "planning_out --> dispatch_in" in text
    no_ffn = {k: v for k, v in tensor_dump.load_rank(str(tmp_path / "d" / "reference"), "chart", 0).items() if k not in ("prefetched_gate", "reduced_grad")}
    assert "prefetch_weight[" not in flowcharts.mermaid(no_ffn) and "combine[" in flowcharts.mermaid(no_ffn)
    assert flowcharts.main([str(tmp_path / "d" / "reference"), "--case", "chart", "--out", str(tmp_path / "c.mmd")]) == 0 and (tmp_path / "c.mmd").exists()

    # what a rank must hold after a dispatch, and where a wrong row is reported
    case = [x for x in cases if x.ranks == 2][1]
    topk = [routing(case, r) for r in range(2)]
    plans = [reference_plan(case, topk, r) for r in range(2)]
    inputs = [make_inputs(case, r) for r in range(2)]
    want = TorchReferenceBackend()
    for r in range(2):
        rows, wrow, source = hl.expected_rows(case, [p["dst"] for p in plans], [i.hidden_sh for i in inputs], [i.route_weights_sk for i in inputs], r)
        filled = int((source >= 0).sum())
        assert filled == sum(int(((p["dst"] >= 0) & (p["dst"] // case.nvs == r)).sum()) for p in plans)
        assert bool((rows[source < 0] == 0).all()) and bool((wrow[source < 0] == 0).all())
        assert hl.first_mismatch(rows, rows.clone(), source) is None
        wrong = rows.clone()
        victim = int(torch.nonzero(source >= 0)[3])
        wrong[victim] = 0
        m = hl.first_mismatch(wrong, rows, source)
        assert m["first_row"] == victim and m["rows_differ"] == 1 and m["got_row_is_zero"] and m["expected_source_rank"] == int(source[victim])
    p = hl.percentiles([float(i) for i in range(1, 101)])
    assert p["count"] == 100 and p["max"] == 100.0 and 50.0 <= p["p50"] <= 51.0 and p["p99"] >= 99.0 and hl.percentiles([])["count"] == 0


def test_model_flow_documents_compare_stage_by_stage(tmp_path):
    """Two runs side by side; a document in the reference's layout (no sequence numbers, no byte counts) is read too."""
    import json

    from tilexr_b200.tools.moonep import model_flow as mf

    def doc(scale, stages):
        ops = [{"stage": s, "phase": "initial_forward", "layer": 0, "latency_us": scale * (i + 1) * 10.0} for i, s in enumerate(stages)]
        return {"ranks": {"0": {"operators": ops}, "1": {"operators": [dict(o, latency_us=o["latency_us"] * 1.5) for o in ops]}}}

    a, b = tmp_path / "a.json", tmp_path / "b.json"
    a.write_text(json.dumps(doc(2.0, mf.FORWARD_STAGES + mf.BACKWARD_STAGES)))
    b.write_text(json.dumps([doc(1.0, mf.FORWARD_STAGES)]))                        # the launcher writes a list of documents
    rows = mf.compare_documents(mf.load_document(str(a)), mf.load_document(str(b)))
    by = {r["stage"]: r for r in rows}
    assert by["planning"]["a_us"] == 30.0 and by["planning"]["b_us"] == 15.0 and abs(by["planning"]["speedup_b_over_a"] - 2.0) < 1e-9   # slowest rank
    assert by["reduce_grad"]["b_us"] is None and by["reduce_grad"]["speedup_b_over_a"] is None
    step = rows[-1]
    assert step["stage"].startswith("step") and abs(step["speedup_b_over_a"] - 2.0) < 1e-9
    assert mf.main(["compare", str(a), str(b)]) == 0 and mf.main(["show", str(a)]) == 0
    bad = tmp_path / "bad.json"
    bad.write_text("{}")
    with pytest.raises(ValueError):
        mf.load_document(str(bad))


def test_orchestrator_script_runs_the_correctness_mode_on_host_memory(tmp_path):
    """`run_moonep.sh N OUT smoke host`: two gloo ranks, the stages through host-memory windows, the verdict table written.  Also
    keeps the script itself sound: every line outside its comments must parse, and nothing runs before the arguments are read."""
    import pathlib
    import subprocess
    import sys

    script = pathlib.Path(__file__).resolve().parents[1] / "tilexr_b200" / "tools" / "run_moonep.sh"
    text = script.read_text().splitlines()
    first_command = next(i for i, line in enumerate(text) if line.strip() and not line.startswith("#"))
    assert text[first_command].strip() == "set -u"
    assert subprocess.run(["bash", "-n", str(script)]).returncode == 0
    env = dict(os.environ, PATH=str(pathlib.Path(sys.executable).parent) + os.pathsep + os.environ.get("PATH", ""),
               PYTHONPATH=str(script.parents[2]) + os.pathsep + os.environ.get("PYTHONPATH", ""))
    r = subprocess.run(["bash", str(script), "2", str(tmp_path), "smoke", "host"], env=env, cwd=str(script.parents[2]), capture_output=True, text=True,
                       timeout=600)
    table = (tmp_path / "correctness.md").read_text()
    assert r.returncode == 0, (r.stdout, r.stderr, (tmp_path / "correctness.err").read_text()[-2000:])
    assert "| smoke_r2 | 0 | pass | - |" in table
    import json

    rows = json.loads((tmp_path / "correctness.json").read_text())
    assert rows and all(x["ok_all_ranks"] for x in rows)


def test_dispatch_hot_loop_on_host_memory(tmp_path):
    """Repeated exact and alternating plans through host-memory windows between two gloo ranks: every launch's rows and route
    weights equal what the plans say, rows that the other plan filled are zero again."""
    import json
    import pathlib
    import subprocess
    import sys

    root = pathlib.Path(__file__).resolve().parents[1]
    out = tmp_path / "hot.json"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nproc-per-node", "2", "--master-addr", "127.0.0.1", "--master-port", str(free_port()),
           "-m", "tilexr_b200.tools.moonep.dispatch_hot_loop", "--backend", "host", "--cases", "smoke", "--iters", "6", "--check-every", "1",
           "--json", str(out)]
    env = dict(os.environ, PYTHONPATH=str(root) + os.pathsep + os.environ.get("PYTHONPATH", ""))
    r = subprocess.run(cmd, cwd=str(root), env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    doc = json.loads(out.read_text())
    assert len(doc) == 1 and doc[0]["ok"] and doc[0]["case"] == "smoke_r2" and len(doc[0]["ranks"]) == 2
    for rank in doc[0]["ranks"]:
        assert rank["failures"] == [] and rank["device_status"] == 0 and rank["latency_us"]["count"] == 12 and rank["bytes"] > 0


def test_route_replay_on_host_memory(tmp_path):
    """Routes captured from two ranks' routers are replayed by the launcher on a host-memory communicator: the operator
    sequence of every layer, forward and backward, with the round trip verified."""
    import json
    import pathlib
    import subprocess
    import sys

    from tilexr_b200.tools.moonep.model_replay import RouteRecorder

    capture = tmp_path / "capture"
    g = torch.Generator().manual_seed(3)
    for rank in range(2):
        rec = RouteRecorder(str(capture), rank, ranks=2, experts=8, prefetch_slots=2, token_padding=4)
        for layer in range(2):
            rec.record(f"layers.{layer}.moe", torch.randint(0, 8, (16, 2), generator=g), hidden=64)
        rec.save()
    root = pathlib.Path(__file__).resolve().parents[1]
    out = tmp_path / "replay.json"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nproc-per-node", "2", "--master-addr", "127.0.0.1", "--master-port", str(free_port()),
           "-m", "tilexr_b200.tools.moonep.launcher", "--mode", "replay", "--backend", "host", "--capture", str(capture), "--iters", "2", "--json", str(out)]
    env = dict(os.environ, PYTHONPATH=str(root) + os.pathsep + os.environ.get("PYTHONPATH", ""), MASTER_PORT=str(free_port()))
    r = subprocess.run(cmd, cwd=str(root), env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    doc = json.loads(out.read_text())
    assert doc["verified"] and doc["backend"] == "host-memory" and [l["layer"] for l in doc["layers"]] == ["layers.0.moe", "layers.1.moe"]
    assert set(doc["total_us"]) == {"planning", "dispatch_fwd", "combine_fwd", "dispatch_bwd", "combine_bwd"} and all(v > 0 for v in doc["total_us"].values())


def test_model_flow_on_host_memory(tmp_path):
    """The operator sequence of a training step (planning, dispatch, prefetch, combine, their backward forms, reduce-grad) issued
    by the launcher on a host-memory communicator: every operator of every layer timed on both ranks, none skipped."""
    import json
    import pathlib
    import subprocess
    import sys

    from tilexr_b200.tools.moonep import model_flow as mf

    root = pathlib.Path(__file__).resolve().parents[1]
    out = tmp_path / "flow.json"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nproc-per-node", "2", "--master-addr", "127.0.0.1", "--master-port", str(free_port()),
           "-m", "tilexr_b200.tools.moonep.launcher", "--mode", "model-flow", "--backend", "host", "--cases", "smoke", "--layers", "2", "--iters", "2",
           "--warmup", "0", "--json", str(out)]
    env = dict(os.environ, PYTHONPATH=str(root) + os.pathsep + os.environ.get("PYTHONPATH", ""))
    r = subprocess.run(cmd, cwd=str(root), env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "| planning | 4 |" in r.stdout and "16750" not in r.stdout            # no published column for the host plumbing
    doc = mf.load_document(str(out))
    assert doc["backend"] == "tilexr-host-memory" and len(doc["operator_order"]) == len(mf.operator_order(2)) == 22
    assert set(doc["ranks"]) == {"0", "1"}
    for entry in doc["ranks"].values():
        ops = entry["operators"]
        assert len(ops) == 22 and not any(o["skipped"] for o in ops) and all(o["latency_us"] > 0 for o in ops)
    med = mf.stage_medians(doc)
    assert set(med) == set(mf.FORWARD_STAGES + mf.BACKWARD_STAGES)
