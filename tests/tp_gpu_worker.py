"""Worker of the multi-GPU tensor-parallel test (launched with torchrun, one rank per GPU)."""
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
os.environ.setdefault("NCCL_NVLS_ENABLE", "0")

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

from tileinfer_b200.engine.llm import LLM  # noqa: E402
from tileinfer_b200.engine.sampling_params import SamplingParams  # noqa: E402


def prompt(n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, 1023, (n,), generator=g).tolist()


def main():
    import faulthandler
    faulthandler.dump_traceback_later(int(os.environ.get("TI_TEST_WATCHDOG_S", "150")), exit=True)   # a stuck rank says where
    fused = os.environ.get("TI_TEST_FUSED", "1") == "1"
    tp = int(os.environ["WORLD_SIZE"])
    llm = LLM("preset:tiny-hybrid-tp", quantization="w8a16", tp_size=tp, num_kvcache_blocks=128, max_num_seqs=8,
              max_model_len=512, max_prefill_chunk_tokens=32, fused_collectives=fused, nccl_timeout=120)
    peer = llm.model_runner.model.peer
    if peer is not None:
        peer.SCRUB_PERIOD = 7          # exercise the periodic buffer scrub many times in this short run
    prompts = [prompt(21, 1), prompt(70, 2), prompt(5, 3)]
    greedy = llm.generate_token_ids(prompts, SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True))
    sampled = llm.generate_token_ids(prompts[:2], SamplingParams(temperature=0.8, top_k=20, max_tokens=8, ignore_eos=True))
    status = llm.model_runner.model.peer_status()
    mine = {"greedy": greedy, "sampled": sampled, "status": status, "scrubs": getattr(peer, "scrubs", 0),
            "graph_launches": llm.model_runner.model.launches_per_decode_step}
    box = [None] * tp
    dist.all_gather_object(box, mine)
    if llm.comm.rank == 0:
        print("TP_RESULT " + json.dumps({"ranks": box, "prompts": prompts, "fused": fused}), flush=True)
    dist.barrier()
    # graphs that captured collectives go before the communicator does
    llm.model_runner.model.graphs.clear()
    torch.cuda.synchronize()
    if llm.model_runner.model.peer is not None:
        llm.model_runner.model.peer.close()
    dist.destroy_process_group()
    faulthandler.cancel_dump_traceback_later()


if __name__ == "__main__":
    main()
