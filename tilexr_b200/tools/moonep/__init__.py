"""MoonEP harness: reference-vs-candidate correctness of the five stages, stage benchmarks, route capture and
replay.  (The reference keeps the same tool set under tools/moonep: benchmark.py, correctness.py,
torch_npu_backend.py, tilexr_backend.py, contracts.py, case_factory.py, planner_reference.py,
expert_forward.py, launcher.py, rendezvous.py, report.py, model_flow.py, model_replay_*.py.)"""
