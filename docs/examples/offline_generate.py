"""Offline generation through the Python API (runs on a CPU box with the reference backend and a tiny model).

    PYTHONPATH=. python docs/examples/offline_generate.py
    PYTHONPATH=. python docs/examples/offline_generate.py --model /models/Qwen3.5-27B-Q4_K_M.gguf --backend cuda_sm100a
"""
import argparse

from hipengine_b200 import LLM, SamplingParams


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="tiny-dense")
    ap.add_argument("--backend", default="cpu_reference")
    a = ap.parse_args()
    llm = LLM(a.model, backend=a.backend, max_active_requests=4, max_sequence_length=512)
    try:
        outs = llm.generate_detailed(["The capital of France is", "1 + 1 ="],
                                     SamplingParams(max_tokens=16, temperature=0.0))
        for o in outs:
            print(repr(o.text), o.finish.reason, f"{o.telemetry.prompt_tokens} prompt tokens")
        print("streamed:", "".join(llm.stream("Once upon a time", SamplingParams(max_tokens=12, temperature=0.7, seed=3))))
        print(llm.fit_context("How long may the answer be?", max_tokens=64))
    finally:
        llm.close()


if __name__ == "__main__":
    main()
