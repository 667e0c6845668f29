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


def leave_between_steps():
    """Rank 1 leaves after a completed request (nothing of its own in flight); rank 0 must learn of it from
    the heartbeat on the host and refuse to launch, with its CUDA context intact."""
    import time
    from tileinfer_b200.parallel.watchdog import PeerLostError
    tp = int(os.environ["WORLD_SIZE"])
    llm = LLM("preset:tiny-hybrid-tp", quantization="w8a16", tp_size=tp, num_kvcache_blocks=128, max_num_seqs=8,
              max_model_len=512, nccl_timeout=60, heartbeat_interval=0.2, heartbeat_timeout=2.0)
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    first = llm.generate_token_ids([prompt(21, 1)], sp)
    torch.cuda.synchronize()
    dist.barrier()
    peer = llm.model_runner.model.peer
    if llm.comm.rank == tp - 1:
        llm.watchdog.stop()
        os._exit(0)
    time.sleep(4.0)
    try:
        llm.generate_token_ids([prompt(9, 2)], sp)
        verdict = "NOT_DETECTED"
    except PeerLostError as e:
        verdict = f"PEER_LOST {e.ranks}"
    ok = float(torch.ones(8, device="cuda").sum()) == 8.0 and llm.model_runner.model.peer_status() == 0
    if llm.comm.rank == 0:
        print(f"LEAVE_RESULT {verdict} context_ok={ok} first_len={len(first[0])}", flush=True)
    llm.model_runner.model.release_graphs()
    peer.close(collective=False)
    os._exit(0)


def main():
    if os.environ.get("TI_TEST_MODE") == "leave":
        return leave_between_steps()
    import faulthandler
    faulthandler.dump_traceback_later(int(os.environ.get("TI_TEST_WATCHDOG_S", "150")), exit=True)   # a stuck rank says where
    fused = os.environ.get("TI_TEST_FUSED", "1") == "1"
    tp = int(os.environ["WORLD_SIZE"])
    preset = "preset:tiny-hybrid-tp8" if tp == 8 else "preset:tiny-hybrid-tp"
    llm = LLM(preset, quantization="w8a16", tp_size=tp, num_kvcache_blocks=128, max_num_seqs=8,
              max_model_len=512, max_prefill_chunk_tokens=32, fused_collectives=fused, nccl_timeout=120)
    peer = llm.model_runner.model.peer
    if peer is not None:
        peer.SCRUB_PERIOD = 7          # exercise the periodic buffer scrub many times in this short run
    prompts = [prompt(21, 1), prompt(70, 2), prompt(5, 3)]
    greedy = llm.generate_token_ids(prompts, SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True))
    sampled = llm.generate_token_ids(prompts[:2], SamplingParams(temperature=0.8, top_k=20, max_tokens=8, ignore_eos=True))
    status = llm.model_runner.model.peer_status()
    mine = {"greedy": greedy, "sampled": sampled, "status": status, "scrubs": getattr(peer, "scrubs", 0),
            "nvls": bool(getattr(peer, "nvls", False)),
            "graph_launches": llm.model_runner.model.launches_per_decode_step}
    box = [None] * tp
    dist.all_gather_object(box, mine)
    if llm.comm.rank == 0:
        print("TP_RESULT " + json.dumps({"ranks": box, "prompts": prompts, "fused": fused}), flush=True)
    dist.barrier()
    # graphs that captured collectives go before the communicator does
    llm.model_runner.model.release_graphs()
    torch.cuda.synchronize()
    if llm.model_runner.model.peer is not None:
        llm.model_runner.model.peer.close()
    dist.destroy_process_group()
    faulthandler.cancel_dump_traceback_later()


if __name__ == "__main__":
    main()
