"""OpenAI-compatible HTTP server: GET /v1/models, POST /v1/chat/completions (JSON or SSE stream).

Same surface as the reference (api_server.py:1-216): stdlib ThreadingHTTPServer, the tokenizer's chat
template, `response_format: {"type": "json_object"}` mapped to JSON mode, one request at a time behind a
lock, HTTP 400 / 404 / 500 mapping, and a tensor-parallel worker loop: rank 0 serves HTTP and hands
every request to the other ranks, which sit in `worker_loop` until a shutdown message arrives.

Differences: the workers receive the prompt together with the COMPLETE SamplingParams (stop strings,
logit bias, allow/deny lists and guided decoding included), because a rank that samples under
different constraints leaves the group out of step (the reference forwards five numeric fields only,
api_server.py:58-61); `finish_reason` is "stop" or "length"; GET /metrics returns the engine counters.
"""
from __future__ import annotations

import argparse
import json
import threading
import time
import uuid
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer

from ..engine.sampling_params import SamplingParams

SHUTDOWN = {"op": "shutdown"}


def build_prompt(tokenizer, messages) -> str:
    try:
        return tokenizer.apply_chat_template(messages, tokenize=False, add_generation_prompt=True)
    except Exception:
        text = "".join(f"{m.get('role', 'user')}: {m.get('content', '')}\n" for m in messages)
        return text + "assistant: "


def make_sampling_params(body: dict) -> SamplingParams:
    kw = {}
    for name, cast in (("temperature", float), ("top_p", float), ("top_k", int), ("max_tokens", int),
                       ("repetition_penalty", float)):
        if body.get(name) is not None:
            kw[name] = cast(body[name])
    if body.get("max_completion_tokens") is not None and "max_tokens" not in kw:
        kw["max_tokens"] = int(body["max_completion_tokens"])
    stop = body.get("stop")
    if stop:
        kw["stop"] = [stop] if isinstance(stop, str) else list(stop)
    for name in ("logit_bias", "allowed_token_ids", "bad_token_ids", "guided_choice", "guided_json", "guided_regex"):
        if body.get(name):
            kw[name] = body[name]
    rf = body.get("response_format")
    if isinstance(rf, dict) and rf.get("type") == "json_object" and "guided_json" not in kw:
        kw["guided_json"] = True
    if body.get("ignore_eos"):
        kw["ignore_eos"] = True
    return SamplingParams(**kw)


class Service:
    """Owns the engine on one rank.  Rank 0 calls `generate` / `stream`; other ranks run `worker_loop`."""

    def __init__(self, llm, model_name: str):
        self.llm = llm
        self.comm = llm.comm
        self.model_name = model_name
        self.lock = threading.Lock()
        self.created = int(time.time())

    # -- tensor-parallel fan-out ------------------------------------------------
    def _announce(self, prompt: str, sp: SamplingParams):
        if self.comm.world_size > 1:
            self.comm.broadcast_object({"op": "generate", "prompt": prompt, "params": sp.to_json()}, src=0)

    def worker_loop(self):
        while True:
            msg = self.comm.broadcast_object(None, src=0)
            if msg is None or msg.get("op") == "shutdown":
                return
            sp = SamplingParams.from_json(msg["params"])
            self.llm.generate([msg["prompt"]], sp)

    def shutdown_workers(self):
        if self.comm.world_size > 1:
            self.comm.broadcast_object(SHUTDOWN, src=0)

    # -- inference ----------------------------------------------------------------
    def generate(self, prompt: str, sp: SamplingParams) -> dict:
        with self.lock:
            self._announce(prompt, sp)
            return self.llm.generate([prompt], sp)[0]

    def stream(self, prompt: str, sp: SamplingParams):
        with self.lock:
            self._announce(prompt, sp)
            for _, text, done in self.llm.generate_stream([prompt], sp):
                yield text, done


def make_handler(svc: Service):
    class Handler(BaseHTTPRequestHandler):
        protocol_version = "HTTP/1.1"

        def log_message(self, fmt, *args):        # quiet, like the reference
            pass

        def _json(self, code: int, obj: dict):
            data = json.dumps(obj).encode()
            self.send_response(code)
            self.send_header("Content-Type", "application/json")
            self.send_header("Content-Length", str(len(data)))
            self.end_headers()
            self.wfile.write(data)

        def _error(self, code: int, msg: str, kind: str = "invalid_request_error"):
            self._json(code, {"error": {"message": msg, "type": kind, "code": code}})

        def do_GET(self):
            if self.path == "/v1/models":
                self._json(200, {"object": "list", "data": [{"id": svc.model_name, "object": "model",
                                                             "created": svc.created, "owned_by": "tileinfer_b200"}]})
            elif self.path in ("/metrics", "/v1/metrics"):
                self._json(200, svc.llm.stats())
            elif self.path == "/health":
                self._json(200, {"status": "ok"})
            else:
                self._error(404, f"unknown path {self.path}", "not_found")

        def do_POST(self):
            if self.path != "/v1/chat/completions":
                return self._error(404, f"unknown path {self.path}", "not_found")
            try:
                n = int(self.headers.get("Content-Length", "0"))
                body = json.loads(self.rfile.read(n) or b"{}")
                messages = body.get("messages")
                if not isinstance(messages, list) or not messages:
                    return self._error(400, "'messages' must be a non-empty list")
                sp = make_sampling_params(body)
                prompt = build_prompt(svc.llm.tokenizer, messages)
            except (ValueError, TypeError, json.JSONDecodeError) as e:
                return self._error(400, str(e))
            rid = "chatcmpl-" + uuid.uuid4().hex[:24]
            try:
                if body.get("stream"):
                    return self._stream(rid, prompt, sp)
                out = svc.generate(prompt, sp)
            except ValueError as e:
                return self._error(400, str(e))
            except Exception as e:            # engine failure
                return self._error(500, f"{type(e).__name__}: {e}", "server_error")
            self._json(200, {
                "id": rid, "object": "chat.completion", "created": int(time.time()), "model": svc.model_name,
                "choices": [{"index": 0, "message": {"role": "assistant", "content": out["text"]},
                             "finish_reason": out.get("finish_reason", "stop")}],
                "usage": {"prompt_tokens": len(out["prompt_token_ids"]), "completion_tokens": len(out["token_ids"]),
                          "total_tokens": len(out["prompt_token_ids"]) + len(out["token_ids"])},
            })

        def _chunk(self, rid, delta, finish=None):
            obj = {"id": rid, "object": "chat.completion.chunk", "created": int(time.time()), "model": svc.model_name,
                   "choices": [{"index": 0, "delta": delta, "finish_reason": finish}]}
            self.wfile.write(f"data: {json.dumps(obj)}\n\n".encode())
            self.wfile.flush()

        def _stream(self, rid, prompt, sp):
            self.send_response(200)
            self.send_header("Content-Type", "text/event-stream")
            self.send_header("Cache-Control", "no-cache")
            self.send_header("Connection", "close")
            self.end_headers()
            try:
                self._chunk(rid, {"role": "assistant"})
                count = 0
                for text, done in svc.stream(prompt, sp):
                    count += 1
                    if text:
                        self._chunk(rid, {"content": text})
                self._chunk(rid, {}, "length" if count >= sp.max_tokens else "stop")
                self.wfile.write(b"data: [DONE]\n\n")
                self.wfile.flush()
            except (BrokenPipeError, ConnectionResetError):
                pass
            self.close_connection = True

    return Handler


def serve(llm, host="127.0.0.1", port=8000, model_name=None, ready=None):
    """Runs the server (rank 0) or the worker loop (other ranks).  Returns when shut down."""
    svc = Service(llm, model_name or llm.config.model)
    if llm.comm.rank != 0:
        svc.worker_loop()
        return None
    httpd = ThreadingHTTPServer((host, port), make_handler(svc))
    httpd.service = svc
    if ready is not None:
        ready(httpd)
    try:
        httpd.serve_forever()
    finally:
        svc.shutdown_workers()
        httpd.server_close()
    return httpd


def add_engine_args(ap: argparse.ArgumentParser):
    ap.add_argument("--model", default="preset:qwen3.6-27b")
    ap.add_argument("--max-num-seqs", type=int, default=64)
    ap.add_argument("--max-model-len", type=int, default=4096)
    ap.add_argument("--gpu-memory-utilization", type=float, default=0.9)
    ap.add_argument("--enforce-eager", action="store_true")
    ap.add_argument("--tp-size", type=int, default=1)
    ap.add_argument("--num-scheduler-steps", type=int, default=1)
    ap.add_argument("--no-prefix-caching", action="store_true")
    ap.add_argument("--quantization", default="w8a16", choices=["w8a16", "bf16"])
    ap.add_argument("--swap-space-gb", type=float, default=0.0)
    ap.add_argument("--device", default="auto")
    ap.add_argument("--heartbeat-interval", type=float, default=0.0,
                    help="seconds between peer heartbeats under tensor parallelism (0: off)")
    ap.add_argument("--weight-cache-dir", default=None, help="keep per-rank quantised shards here between starts")


def engine_kwargs(args) -> dict:
    return dict(max_num_seqs=args.max_num_seqs, max_model_len=args.max_model_len,
                gpu_memory_utilization=args.gpu_memory_utilization, enforce_eager=args.enforce_eager,
                tp_size=args.tp_size, num_scheduler_steps=args.num_scheduler_steps,
                enable_prefix_caching=not args.no_prefix_caching, quantization=args.quantization,
                swap_space_bytes=int(args.swap_space_gb * (1 << 30)), device=args.device,
                weight_cache_dir=args.weight_cache_dir, heartbeat_interval=args.heartbeat_interval)


def main(argv=None):
    ap = argparse.ArgumentParser(description="tileinfer_b200 OpenAI-compatible server")
    add_engine_args(ap)
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=8000)
    args = ap.parse_args(argv)
    from ..engine.llm import LLM
    llm = LLM(args.model, **engine_kwargs(args))
    if llm.comm.rank == 0:
        print(f"serving {args.model} on http://{args.host}:{args.port}", flush=True)
    try:
        serve(llm, args.host, args.port)
    except KeyboardInterrupt:
        pass
    finally:
        llm.close()         # every rank gets here: the workers leave their loop when rank 0 shuts them down


if __name__ == "__main__":
    main()
