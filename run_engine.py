"""Command-line generation (reference: run_engine.py:27-94): builds an LLM, runs one generate, rank 0 prints.

    python run_engine.py --model preset:tiny-hybrid --prompt "hello" --max-tokens 32
    torchrun --nproc-per-node 2 run_engine.py --tp-size 2 --prompt "hello"
"""
import argparse
import json

from tileinfer_b200.engine.llm import LLM
from tileinfer_b200.engine.sampling_params import SamplingParams
from tileinfer_b200.server.api_server import add_engine_args, engine_kwargs


def main(argv=None):
    ap = argparse.ArgumentParser()
    add_engine_args(ap)
    ap.add_argument("--prompt", default="Hello")
    ap.add_argument("--temperature", type=float, default=0.6)
    ap.add_argument("--top-p", type=float, default=1.0)
    ap.add_argument("--top-k", type=int, default=-1)
    ap.add_argument("--max-tokens", type=int, default=64)
    ap.add_argument("--guided-json", action="store_true")
    ap.add_argument("--guided-regex", default=None)
    ap.add_argument("--guided-choice", nargs="*", default=[])
    ap.add_argument("--stats", action="store_true")
    args = ap.parse_args(argv)
    llm = LLM(args.model, **engine_kwargs(args))
    sp = SamplingParams(temperature=args.temperature, top_p=args.top_p, top_k=args.top_k, max_tokens=args.max_tokens,
                        guided_json=True if args.guided_json else None, guided_regex=args.guided_regex,
                        guided_choice=list(args.guided_choice))
    out = llm.generate([args.prompt], sp)[0]
    if llm.comm.rank == 0:
        print(out["text"])
        if args.stats:
            print(json.dumps(llm.stats(), indent=1))
    llm.close()
    return out


if __name__ == "__main__":
    main()
