"""Interpreter start-up hook: put this folder on PYTHONPATH and set VLLM_TILEXR_COLLECTIVES=1, and every Python process of a
vLLM deployment (the engine and its workers) routes its CUDA communicator through this library's collectives without a change
to vLLM or to the launch script (the reference ships the same hook for its vLLM-Ascend glue:
integrations/vllm_ascend/sitecustomize.py).  Any problem leaves vLLM on its stock path; TILEXR_VLLM_TRACE=1 says why."""
import os
import sys


def _on(name: str) -> bool:
    return os.environ.get(name, "0").strip().lower() in ("1", "true", "yes", "on")


if _on("VLLM_TILEXR_COLLECTIVES") or _on("VLLM_ASCEND_TILEXR_COLLECTIVES"):
    try:
        from tilexr_b200.integrations.vllm_collectives import autopatch

        autopatch()
    except Exception as exc:  # never break the interpreter's start
        if _on("TILEXR_VLLM_TRACE"):
            print(f"[tilexr-vllm] start-up hook left the stock path in place: {type(exc).__name__}: {exc}", file=sys.stderr)
