"""HTTP surface: OpenAI- and Anthropic-compatible inference, control API, Prometheus metrics.

Route and payload parity with the reference server (``mfq/server/api/routes/openai.py:28-157``,
``anthropic.py:20-55``, ``runtime.py``, ``docs/api/http.md``):

* ``GET /health``, ``GET /v1``, ``GET /v1/models``, ``GET /v1/models/{id}``
* ``POST /v1/chat/completions`` -- JSON or SSE ``chat.completion.chunk`` stream; accepts ``max_tokens``,
  ``temperature``, ``top_p``, ``top_k``, ``presence_penalty``, ``frequency_penalty``, ``repetition_penalty``,
  ``seed``, ``stop``, ``stream``, ``priority``, ``timeout_seconds``, ``session_id`` (KV snapshot reuse across turns), ``enable_mtp``, ``mtp_max_draft_tokens``
* ``POST /v1/messages`` (Anthropic; stream or not), ``POST /v1/messages/count_tokens`` -> 501
* ``GET /metrics`` (text 0.0.4), ``/api/v1/runtime/{status,instances,concurrency}``,
  ``POST /api/v1/models/{load,unload}``
* bearer / ``x-api-key`` auth when a key is configured (``/health`` stays open)
* error envelope ``{"error": {"code", "message", "retryable", "details"}}`` with 429 ``runtime_queue_full``,
  503 ``runtime_queue_timeout``, 504 ``runtime_deadline_exceeded``.
"""

from __future__ import annotations

import asyncio
import json
import queue
import time
import uuid
from pathlib import Path

from fastapi import FastAPI, Request as HttpRequest, WebSocket, WebSocketDisconnect
from fastapi.responses import JSONResponse, PlainTextResponse, StreamingResponse

from ..engine.scheduler import BackendFailure, QueueFull, SamplingParams
from .service import ModelService
from .tokenizer import _content_text


def error_response(status: int, code: str, message: str, retryable: bool = False, details=None) -> JSONResponse:
    return JSONResponse({"error": {"code": code, "message": message, "retryable": retryable, "details": details or {}}},
                        status_code=status)


_ERROR_STATUS = {"runtime_queue_full": (429, True), "runtime_queue_timeout": (503, True),
                 "runtime_deadline_exceeded": (504, False), "backend_failure": (500, True), "error": (400, False)}


def _params_from(body: dict, stop_ids: tuple[int, ...]) -> SamplingParams:
    return SamplingParams(
        max_tokens=int(body.get("max_tokens") or body.get("max_completion_tokens") or 256),
        temperature=float(body.get("temperature", 0.0) or 0.0), top_k=int(body.get("top_k", 0) or 0),
        top_p=float(body.get("top_p", 1.0) or 1.0), presence_penalty=float(body.get("presence_penalty", 0.0) or 0.0),
        frequency_penalty=float(body.get("frequency_penalty", 0.0) or 0.0),
        repetition_penalty=float(body.get("repetition_penalty", 1.0) or 1.0), seed=int(body.get("seed", 0) or 0),
        stop_token_ids=stop_ids, enable_mtp=bool(body.get("enable_mtp", False)),
        mtp_max_draft_tokens=int(body.get("mtp_max_draft_tokens", 3) or 3),
        response_format=_response_format(body.get("response_format")),
        logit_bias={int(k): float(v) for k, v in (body.get("logit_bias") or {}).items()} or None)


def _response_format(value):
    """OpenAI ``response_format``: ``{"type": "json_object" | "json_schema" | "text"}`` -> what the engine constrains
    on (None for free text).  A schema is held to "a JSON object"; its keys are not enforced token by token."""
    kind = value.get("type") if isinstance(value, dict) else value
    if kind in (None, "", "text"):
        return None
    if kind not in ("json_object", "json_schema"):
        raise ValueError(f"unsupported response_format type {kind!r}")
    return {"type": kind}


class _Stream:
    """Turns scheduler events of one request into decoded text pieces, honouring stop strings."""

    def __init__(self, service: ModelService, model, req, events, stop: list[str]) -> None:
        self.service, self.model, self.req, self.events, self.stop = service, model, req, events, stop
        self.ids: list[int] = []
        self.text = ""
        self.finish: str | None = None
        self.error_code: str | None = None

    async def pieces(self):
        loop = asyncio.get_running_loop()
        while True:
            try:
                ev = await loop.run_in_executor(None, self.events.get, True, 0.25)
            except queue.Empty:
                continue
            if ev.kind == "token":
                if ev.token in self.req.params.stop_token_ids:
                    continue
                self.ids.append(ev.token)
                full = self.model.tokenizer.decode(self.ids)
                piece, self.text = full[len(self.text):], full
                cut = min((self.text.find(s) for s in self.stop if s and s in self.text), default=-1)
                if cut >= 0:
                    keep = cut - (len(self.text) - len(piece))
                    if keep > 0:
                        yield piece[:keep]
                    self.text = self.text[:cut]
                    self.finish = "stop"
                    self.service.cancel(self.model, self.req.id)
                    self.service.record_completion(self.model, self.req, "ok")
                    return
                if piece:
                    yield piece
            elif ev.kind == "completed":
                self.finish = self.finish or ("stop" if ev.finish_reason in ("stop", "cancelled") else "length")
                self.service.record_completion(self.model, self.req, "cancelled" if ev.finish_reason == "cancelled" else "ok")
                return
            elif ev.kind == "failed":
                self.error_code = ev.error_code or "error"
                result = "timeout" if "deadline" in self.error_code or "timeout" in self.error_code else "error"
                self.service.record_completion(self.model, self.req, result)
                return


def create_app(service: ModelService, api_key=None, sessions=None, cluster=None, hardware=None, policies=None,
               catalog=None) -> FastAPI:
    """``api_key``: one key with every scope, or a :class:`~mfq_b200.server.auth.KeyStore`; ``sessions``: a :class:`~mfq_b200.server.sessions.SessionStore` (in-memory when omitted); ``cluster``: a
    :class:`~mfq_b200.server.cluster.ClusterBackend` whose peers serve models that are not loaded here; ``hardware``:
    a :class:`~mfq_b200.server.hardware.HardwareMonitor`; ``catalog``: a :class:`~mfq_b200.server.catalog.ModelCatalog`
    of artifacts on disk (the ``/api/v1/catalog`` routes)."""
    from .hardware import HardwareMonitor
    from .sessions import SessionStore
    from contextlib import asynccontextmanager
    from .jobs import JobManager
    from .policies import PolicyStore
    jobs = JobManager()
    instance_id, started_at = uuid.uuid4().hex, time.time()
    policies = policies if policies is not None else PolicyStore()
    for _lm in service.models.values():
        policies.apply_concurrency(_lm.name, _lm.scheduler)

    @asynccontextmanager
    async def lifespan(_app):
        history.start()
        yield
        history.stop()
        jobs.shutdown()  # child processes started through the jobs API end with the server

    app = FastAPI(title="mfq-b200", version="0.1.0", lifespan=lifespan)
    app.state.service = service
    app.state.jobs = jobs
    app.state.cluster = cluster
    monitor = hardware if hardware is not None else HardwareMonitor()
    from .hardware import ResourceHistory
    history = ResourceHistory(monitor)
    app.state.resource_history = history
    store = sessions if sessions is not None else SessionStore()
    app.state.sessions = store

    from .auth import KeyStore, required_scope
    keys = api_key if isinstance(api_key, KeyStore) else KeyStore()
    if isinstance(api_key, str) and api_key:
        keys.add(api_key, ("admin",), name="startup key")
    app.state.keys = keys

    @app.middleware("http")
    async def auth(request: HttpRequest, call_next):
        scope = required_scope(request.method, request.url.path)
        if scope is not None and keys.enforce:
            supplied = request.headers.get("x-api-key")
            header = request.headers.get("authorization", "")
            if header.lower().startswith("bearer "):
                supplied = header[7:].strip()
            if keys.scopes_of(supplied) is None:
                return error_response(401, "unauthorized", "missing or invalid API key")
            if not keys.allows(supplied, scope):
                return error_response(403, "forbidden", f"this key lacks the {scope!r} scope")
        response = await call_next(request)
        response.headers["x-content-type-options"] = "nosniff"
        return response

    @app.get("/health")
    async def health():
        names = list(service.models)
        ok = all(lm.scheduler.healthy for lm in service.models.values())
        return {"status": "ok" if ok else "degraded", "model": names[-1] if names else None, "models": names}

    @app.get("/v1")
    async def v1_root():
        return {"object": "api", "endpoints": ["/v1/models", "/v1/chat/completions", "/v1/messages"]}

    def _model_card(lm):
        return {"id": lm.name, "object": "model", "created": int(lm.loaded_at), "owned_by": "mfq"}

    @app.get("/v1/models")
    async def models():
        cards = [_model_card(lm) for lm in service.models.values()]
        if cluster is not None:
            local = {c["id"] for c in cards}
            cards += [{"id": m, "object": "model", "created": 0, "owned_by": "mfq-cluster"} for m in cluster.models() if m not in local]
        return {"object": "list", "data": cards}

    @app.get("/v1/models/{model_id}")
    async def model(model_id: str):
        if model_id not in service.models:
            return error_response(404, "model_not_found", f"model {model_id!r} is not loaded")
        return _model_card(service.models[model_id])

    async def _start(body: dict, messages: list[dict], stop: list[str]):
        try:
            lm = service.resolve(body.get("model"))
        except KeyError as exc:
            return None, error_response(404, "model_not_found", f"model {exc.args[0]!r} is not loaded")
        from . import tools as tool_ops
        template_vars = dict(body.get("chat_template_kwargs") or {})
        if body.get("enable_thinking") is not None:  # request-level switch of reasoning, as the templates spell it
            template_vars["enable_thinking"] = bool(body["enable_thinking"])
        prompt = lm.tokenizer.apply_chat_template(tool_ops.with_tools(messages, tool_ops.normalise(body.get("tools"))),
                                                  add_generation_prompt=True, **template_vars)
        ids = lm.tokenizer.encode(prompt)
        if not ids:
            return None, error_response(400, "invalid_request", "empty prompt")
        try:
            merged = policies.request_defaults(lm.name, body)
            if "profile_defaults" not in lm.meta:
                from ..formats import runtime_profile as rp
                try:
                    lm.meta["profile_defaults"] = rp.checkpoint_defaults(lm.meta)
                except (ValueError, OSError):
                    lm.meta["profile_defaults"] = {}
            merged = {**lm.meta["profile_defaults"], **{k: v for k, v in merged.items() if v is not None}}
            params = _params_from(merged, tuple(lm.tokenizer.stop_ids))
        except (TypeError, ValueError) as exc:
            return None, error_response(400, "invalid_request", str(exc))
        try:
            req, events = await asyncio.get_running_loop().run_in_executor(
                None, lambda: service.submit(lm, ids, params, priority=int(body.get("priority", 0) or 0),
                                             timeout_seconds=body.get("timeout_seconds"),
                                             session=body.get("session_id")))
        except QueueFull as exc:
            return None, error_response(429, "runtime_queue_full", str(exc), retryable=True)
        except BackendFailure as exc:
            return None, error_response(500, "backend_failure", str(exc), retryable=True)
        return (_Stream(service, lm, req, events, stop), lm, ids), None

    def _failure(stream: _Stream):
        status, retry = _ERROR_STATUS.get(stream.error_code, (500, False))
        return error_response(status, stream.error_code, "generation failed", retryable=retry)

    async def _remote(path: str, body: dict):
        """Models that only a cluster peer serves: forward the request as it is (streaming bodies line by line)."""
        from .cluster import NoPeer
        loop = asyncio.get_running_loop()
        try:
            status, out, _peer = await loop.run_in_executor(None, lambda: cluster.forward(path, body, bool(body.get("stream"))))
        except NoPeer:
            return error_response(503, "no_healthy_peer", f"no healthy cluster peer serves {body.get('model')!r}", retryable=True)
        if body.get("stream") and status < 400:
            return StreamingResponse(iter(out), media_type="text/event-stream")
        if body.get("stream"):
            out = json.loads(b"".join(out) or b"{}")
        return JSONResponse(out, status_code=status)

    def _is_remote(body: dict) -> bool:
        name = body.get("model")
        return bool(cluster is not None and name and name not in service.models and service.loader is None
                    and name in cluster.models())

    @app.post("/v1/chat/completions")
    async def chat(request: HttpRequest):
        body = await request.json()
        if _is_remote(body):
            return await _remote("/v1/chat/completions", body)
        messages = body.get("messages") or []
        if not messages:
            return error_response(400, "invalid_request", "messages must not be empty")
        stop = body.get("stop") or []
        stop = [stop] if isinstance(stop, str) else list(stop)
        started, err = await _start(body, messages, stop)
        if err is not None:
            return err
        stream, lm, ids = started
        cid, created = f"chatcmpl-{uuid.uuid4().hex[:24]}", int(time.time())

        def usage():
            return {"prompt_tokens": len(ids), "completion_tokens": len(stream.ids), "total_tokens": len(ids) + len(stream.ids)}

        if body.get("stream"):
            async def sse():
                def chunk(delta, finish=None, extra=None):
                    d = {"id": cid, "object": "chat.completion.chunk", "created": created, "model": lm.name,
                         "choices": [{"index": 0, "delta": delta, "finish_reason": finish}]}
                    if extra:
                        d.update(extra)
                    return f"data: {json.dumps(d)}\n\n"
                yield chunk({"role": "assistant", "content": ""})
                async for piece in stream.pieces():
                    yield chunk({"content": piece})
                if stream.error_code:
                    yield f"data: {json.dumps({'error': {'code': stream.error_code, 'message': 'generation failed'}})}\n\n"
                else:
                    extra = {"usage": usage()} if (body.get("stream_options") or {}).get("include_usage") else None
                    yield chunk({}, stream.finish or "stop", extra)
                yield "data: [DONE]\n\n"
            return StreamingResponse(sse(), media_type="text/event-stream")
        async for _ in stream.pieces():
            pass
        if stream.error_code:
            return _failure(stream)
        from . import tools as tool_ops
        reasoning, answer = tool_ops.split_reasoning(stream.text)
        message, finish = {"role": "assistant", "content": answer}, stream.finish or "stop"
        if reasoning is not None:
            message["reasoning_content"] = reasoning
        if body.get("tools"):
            text, calls = tool_ops.extract(answer)
            if calls:
                message.update(content=text or None, tool_calls=tool_ops.openai_calls(calls))
                finish = "tool_calls"
        return {"id": cid, "object": "chat.completion", "created": created, "model": lm.name,
                "choices": [{"index": 0, "message": message, "finish_reason": finish}], "usage": usage()}

    @app.post("/v1/messages")
    async def anthropic_messages(request: HttpRequest):
        body = await request.json()
        messages = list(body.get("messages") or [])
        if not messages:
            return error_response(400, "invalid_request", "messages must not be empty")
        if body.get("system"):
            messages = [{"role": "system", "content": _content_text(body["system"])}] + messages
        started, err = await _start(body, messages, list(body.get("stop_sequences") or []))
        if err is not None:
            return err
        stream, lm, ids = started
        mid = f"msg_{uuid.uuid4().hex[:24]}"

        def stop_reason():
            return "end_turn" if stream.finish == "stop" else "max_tokens"

        if body.get("stream"):
            async def sse():
                def ev(name, data):
                    return f"event: {name}\ndata: {json.dumps(data)}\n\n"
                yield ev("message_start", {"type": "message_start", "message": {
                    "id": mid, "type": "message", "role": "assistant", "model": lm.name, "content": [],
                    "stop_reason": None, "usage": {"input_tokens": len(ids), "output_tokens": 0}}})
                yield ev("content_block_start", {"type": "content_block_start", "index": 0, "content_block": {"type": "text", "text": ""}})
                async for piece in stream.pieces():
                    yield ev("content_block_delta", {"type": "content_block_delta", "index": 0, "delta": {"type": "text_delta", "text": piece}})
                yield ev("content_block_stop", {"type": "content_block_stop", "index": 0})
                if stream.error_code:
                    yield ev("error", {"type": "error", "error": {"type": stream.error_code, "message": "generation failed"}})
                else:
                    yield ev("message_delta", {"type": "message_delta", "delta": {"stop_reason": stop_reason(), "stop_sequence": None},
                                               "usage": {"output_tokens": len(stream.ids)}})
                yield ev("message_stop", {"type": "message_stop"})
            return StreamingResponse(sse(), media_type="text/event-stream")
        async for _ in stream.pieces():
            pass
        if stream.error_code:
            return _failure(stream)
        content, reason = [{"type": "text", "text": stream.text}], stop_reason()
        if body.get("tools"):
            from . import tools as tool_ops
            text, calls = tool_ops.extract(stream.text)
            if calls:
                content, reason = tool_ops.anthropic_blocks(text, calls), "tool_use"
        return {"id": mid, "type": "message", "role": "assistant", "model": lm.name,
                "content": content, "stop_reason": reason, "stop_sequence": None,
                "usage": {"input_tokens": len(ids), "output_tokens": len(stream.ids)}}

    @app.post("/v1/messages/count_tokens")
    async def count_tokens():
        return error_response(501, "not_implemented", "count_tokens is not provided")

    @app.get("/metrics")
    async def metrics():
        return PlainTextResponse(service.metrics.render(service), media_type="text/plain; version=0.0.4")

    @app.get("/api/v1/runtime/status")
    async def runtime_status():
        return service.status()

    @app.get("/api/v1/runtime/instances")
    async def runtime_instances():
        return service.status()["instances"]

    # ---- jobs (quantize / eval / inspect ... as child processes) -----------------------------------------------------
    @app.get("/api/v1/jobs")
    async def list_jobs():
        return {"jobs": [j.describe(0) for j in jobs.jobs.values()]}

    @app.post("/api/v1/jobs")
    async def start_job(request: HttpRequest):
        body = await request.json()
        try:
            job = jobs.submit(str(body.get("kind", "")), list(body.get("args") or []))
        except ValueError as exc:
            return error_response(400, "invalid_request", str(exc))
        except RuntimeError as exc:
            return error_response(429, "too_many_jobs", str(exc), retryable=True)
        return JSONResponse(job.describe(), status_code=202)

    @app.get("/api/v1/jobs/{jid}")
    async def get_job(jid: str):
        job = jobs.jobs.get(jid)
        return job.describe() if job is not None else error_response(404, "job_not_found", f"no job {jid!r}")

    @app.post("/api/v1/jobs/{jid}/cancel")
    async def cancel_job(jid: str):
        return {"cancelled": jobs.cancel(jid)}

    @app.delete("/api/v1/jobs/{jid}")
    async def delete_job(jid: str):
        return {"deleted": jobs.delete(jid)}

    @app.get("/api/v1/auth/keys")
    async def list_keys():
        return {"keys": keys.listing()}

    @app.post("/api/v1/auth/keys")
    async def create_key(request: HttpRequest):
        body = await request.json()
        try:
            key, rec = keys.create(tuple(body.get("scopes") or ("inference",)), str(body.get("name", "")))
        except ValueError as exc:
            return error_response(400, "invalid_request", str(exc))
        return {"key": key, **rec}  # the only time the key itself is shown

    @app.delete("/api/v1/auth/keys/{key_id}")
    async def revoke_key(key_id: str):
        try:
            return {"revoked": keys.revoke(key_id)}
        except ValueError as exc:
            return error_response(409, "last_admin_key", str(exc))

    @app.get("/api/v1/hardware")
    async def hardware_snapshot():
        return monitor.snapshot()

    @app.get("/api/v1/hardware/history")
    async def hardware_history(last: int | None = None):
        """Timeline of GPU and host usage (one sample per second while the server runs; a first call takes one)."""
        if not history.samples:
            history.sample()
        return history.history(last)

    @app.get("/api/v1/cluster")
    async def cluster_status():
        return {"peers": cluster.status() if cluster is not None else []}

    @app.get("/api/v1/runtime/cache")
    async def cache_entries():
        out = []
        for lm in service.models.values():
            eng = getattr(lm, "engine", None)
            sc, pc = getattr(eng, "session_cache", None), getattr(eng, "prefix_cache", None)
            out.append({"model": lm.name,
                        "sessions": {"entries": len(sc.entries), "bytes": sc.bytes, **sc.stats} if sc is not None else None,
                        "prefix": dict(getattr(eng, "prefix_stats", {})) if pc is not None else None})
        return {"caches": out}

    @app.post("/api/v1/runtime/cache/purge")
    async def cache_purge(request: HttpRequest):
        body = await request.json()
        dropped = 0
        for lm in service.models.values():
            sc = getattr(getattr(lm, "engine", None), "session_cache", None)
            if sc is None or body.get("model") not in (None, lm.name):
                continue
            for sid in [body["session"]] if body.get("session") else list(sc.entries):
                if sid in sc.entries:
                    sc.drop(sid)
                    dropped += 1
        return {"dropped": dropped}

    @app.get("/api/v1/runtime/concurrency")
    async def concurrency():
        return [{"model": lm.name, "batch_capacity": lm.request_capacity, "max_queue": lm.scheduler.max_queue,
                 "queue_timeout": lm.scheduler.queue_timeout} for lm in service.models.values()]

    @app.get("/api/v1/runtime/policies")
    async def list_policies():
        return {"policies": policies.all(), "sections": {k: sorted(v) for k, v in __import__("mfq_b200.server.policies", fromlist=["SECTIONS"]).SECTIONS.items()}}

    @app.get("/api/v1/runtime/policies/{model}")
    async def get_policy(model: str):
        return {"model": model, "policy": policies.get(model)}

    @app.put("/api/v1/runtime/policies/{model}")
    async def put_policy(model: str, request: HttpRequest):
        try:
            clean = policies.put(model, await request.json())
        except ValueError as exc:
            return error_response(400, "invalid_request", str(exc))
        if model in service.models:
            policies.apply_concurrency(model, service.models[model].scheduler)
        return {"model": model, "policy": clean}

    @app.post("/api/v1/models/load")
    async def load_model(request: HttpRequest):
        body = await request.json()
        try:
            lm = await asyncio.get_running_loop().run_in_executor(None, service.load, body.get("model", ""))
        except KeyError:
            return error_response(404, "model_not_found", "unknown model and no loader configured")
        policies.apply_concurrency(lm.name, lm.scheduler)
        return {"model": lm.name, "instance": lm.instance}

    @app.post("/api/v1/models/unload")
    async def unload_model(request: HttpRequest):
        body = await request.json()
        return {"unloaded": service.unload(body.get("model", ""))}

    # ---- catalog of artifacts on disk ----------------------------------------------------------------------------
    from .catalog import ArtifactNotFound, ModelCatalog
    cat = catalog if catalog is not None else ModelCatalog()
    app.state.catalog = cat

    @app.get("/api/v1/catalog")
    async def catalog_list():
        return {"roots": cat.roots, "models": cat.listing()}

    @app.post("/api/v1/catalog/scan")
    async def catalog_scan(request: HttpRequest):
        body = await request.json() if await request.body() else {}
        for root in body.get("roots", []):
            cat.add_root(root)
        return await asyncio.get_running_loop().run_in_executor(None, cat.scan)

    @app.put("/api/v1/catalog/{ident}/aliases/{name}")
    async def catalog_alias(ident: str, name: str):
        try:
            cat.alias(name, ident)
        except ArtifactNotFound:
            return error_response(404, "model_not_found", f"no catalog entry {ident!r}")
        return {"id": ident, "aliases": cat.resolve(ident).aliases}

    @app.delete("/api/v1/catalog/{ident}")
    async def catalog_remove(ident: str, purge: bool = False):
        """Forget an entry; ``purge=true`` also deletes its files, which must lie under one of the catalog's roots."""
        if not purge:
            return {"removed": cat.remove(ident)}
        try:
            art = cat.resolve(ident)
        except ArtifactNotFound:
            return error_response(404, "model_not_found", f"no catalog entry {ident!r}")
        if any(name in (art.id, *art.aliases) for name in service.models):
            return error_response(409, "model_loaded", f"{ident!r} is loaded; unload it first")
        try:
            freed = cat.purge(art.id)
        except PermissionError as exc:
            return error_response(403, "outside_catalog_roots", str(exc))
        return {"removed": True, "purged": True, "freed_bytes": freed}

    @app.get("/api/v1/catalog/{ident}/analysis")
    async def catalog_analysis(ident: str, batch: int = 1, context: int = 4096, tensor_parallel: int = 1):
        """Composition of a checkpoint (bytes and bits per weight per family and group), parameter counts (total and
        active per token) and the device memory a deployment of ``batch`` x ``context`` needs per GPU."""
        from .analysis import analyse_artifact
        try:
            art = cat.resolve(ident)
        except ArtifactNotFound:
            return error_response(404, "model_not_found", f"no catalog entry {ident!r}")
        if batch < 1 or context < 1 or tensor_parallel < 1:
            return error_response(400, "invalid_request", "batch, context and tensor_parallel must be positive")
        fn = lambda: analyse_artifact(art, batch=batch, context=context, tensor_parallel=tensor_parallel)
        return await asyncio.get_running_loop().run_in_executor(None, fn)

    @app.get("/api/v1/runtime/stats")
    async def runtime_stats():
        """Request counters and latency / throughput quantiles per model, from the metrics histograms."""
        from .analysis import serving_stats
        return serving_stats(service.metrics)

    # ---- realtime: one WebSocket, many generations ------------------------------------------------------------------

    @app.websocket("/api/v1/realtime")
    async def realtime(ws: WebSocket):
        """Frames in: ``{"type": "generate", "id", "model", "messages", sampling fields...}``, ``{"type": "cancel", "id"}``,
        ``{"type": "ping"}``.  Frames out: ``started``, ``delta`` (text pieces), ``done`` (finish reason + usage), ``error``,
        ``pong``.  Several generations may run at once on one socket; closing the socket cancels them all."""
        if keys.enforce:
            supplied = ws.headers.get("x-api-key") or ws.query_params.get("api_key")
            header = ws.headers.get("authorization", "")
            if header.lower().startswith("bearer "):
                supplied = header[7:].strip()
            if keys.scopes_of(supplied) is None or not keys.allows(supplied, "inference"):
                await ws.close(code=4401)
                return
        await ws.accept()
        running: dict[str, tuple] = {}
        send_lock = asyncio.Lock()

        async def send(frame: dict) -> None:
            async with send_lock:
                await ws.send_text(json.dumps(frame))

        async def pump(rid: str, stream, lm, ids) -> None:
            try:
                async for piece in stream.pieces():
                    await send({"type": "delta", "id": rid, "text": piece})
                if stream.error_code:
                    await send({"type": "error", "id": rid, "code": stream.error_code})
                else:
                    await send({"type": "done", "id": rid, "finish_reason": stream.finish or "stop", "text": stream.text,
                                "usage": {"prompt_tokens": len(ids), "completion_tokens": len(stream.ids)}})
            finally:
                running.pop(rid, None)

        try:
            while True:
                try:
                    frame = json.loads(await ws.receive_text())
                except json.JSONDecodeError:
                    await send({"type": "error", "code": "invalid_request", "message": "frames are JSON objects"})
                    continue
                kind, rid = frame.get("type"), str(frame.get("id", ""))
                if kind == "ping":
                    await send({"type": "pong"})
                elif kind == "cancel":
                    entry = running.get(rid)
                    if entry is not None:
                        service.cancel(entry[1], entry[2].id)
                    await send({"type": "cancelling" if entry else "error", "id": rid, **({} if entry else {"code": "unknown_id"})})
                elif kind == "generate":
                    if not rid or rid in running:
                        await send({"type": "error", "id": rid, "code": "invalid_request", "message": "id missing or in use"})
                        continue
                    stop = frame.get("stop") or []
                    started, err = await _start(frame, frame.get("messages") or [], [stop] if isinstance(stop, str) else list(stop))
                    if err is not None:
                        payload = json.loads(err.body)
                        await send({"type": "error", "id": rid, **payload.get("error", {})})
                        continue
                    stream, lm, ids = started
                    running[rid] = (asyncio.create_task(pump(rid, stream, lm, ids)), lm, stream.req)
                    await send({"type": "started", "id": rid, "model": lm.name, "prompt_tokens": len(ids)})
                else:
                    await send({"type": "error", "id": rid, "code": "invalid_request", "message": f"unknown frame type {kind!r}"})
        except WebSocketDisconnect:
            pass
        finally:
            for task, lm, req in list(running.values()):
                service.cancel(lm, req.id)
                task.cancel()

    # ---- sessions (chat history kept by the server for its clients) ----------------------------------------------
    @app.get("/api/v1/sessions")
    async def list_sessions():
        return {"sessions": store.list()}

    @app.post("/api/v1/sessions")
    async def create_session(request: HttpRequest):
        body = await request.json() if await request.body() else {}
        return store.create(body.get("title", ""), body.get("model"), body.get("meta"))

    @app.get("/api/v1/sessions/{sid}")
    async def get_session(sid: str):
        s = store.get(sid)
        return s if s is not None else error_response(404, "session_not_found", f"no session {sid!r}")

    @app.post("/api/v1/sessions/{sid}/messages")
    async def append_message(sid: str, request: HttpRequest):
        body = await request.json()
        try:
            seq = store.append(sid, body.get("role", "user"), body.get("content", ""), body.get("meta"))
        except KeyError:
            return error_response(404, "session_not_found", f"no session {sid!r}")
        return {"seq": seq}

    @app.patch("/api/v1/sessions/{sid}")
    async def rename_session(sid: str, request: HttpRequest):
        body = await request.json()
        ok = store.rename(sid, body.get("title", ""))
        return {"renamed": True} if ok else error_response(404, "session_not_found", f"no session {sid!r}")

    @app.delete("/api/v1/sessions/{sid}")
    async def delete_session(sid: str):
        return {"deleted": store.delete(sid)}

    @app.get("/health/identity")
    async def health_identity():
        """Who answers here: package version, a process-lifetime instance id, the models it serves.  A cluster peer
        list uses it to tell a restarted server from the one it knew."""
        from .. import __version__
        return {"service": "mfq_b200", "version": __version__, "instance_id": instance_id,
                "started_at": started_at, "models": sorted(service.models)}

    @app.get("/api/v1/models/{model}/cache-profile")
    async def get_cache_profile(model: str):
        """Per-expert heat of a model whose routed experts sit behind an HBM slot arena (what ``--moe-cache-profile``
        saves and a later start warms the arena from)."""
        from ..engine import moe_cache_profile as mcp
        lm = service.models.get(model)
        if lm is None:
            return error_response(404, "model_not_found", f"model {model!r} is not loaded")
        inner = getattr(getattr(lm, "engine", None), "model", None) or getattr(getattr(getattr(lm, "engine", None), "engine", None), "model", None)
        if inner is None or not getattr(inner, "residencies", lambda: [])():
            return error_response(409, "no_expert_cache", f"model {model!r} keeps every expert resident: there is no cache to profile")
        return await asyncio.get_running_loop().run_in_executor(None, service.call, lm, lambda _m: mcp.collect(inner, model))

    @app.post("/api/v1/models/{model}/cache-profile")
    async def apply_cache_profile(model: str, request: HttpRequest):
        """Warm the expert arena from a profile (the body is what the GET returns)."""
        from ..engine import moe_cache_profile as mcp
        lm = service.models.get(model)
        if lm is None:
            return error_response(404, "model_not_found", f"model {model!r} is not loaded")
        inner = getattr(getattr(lm, "engine", None), "model", None)
        if inner is None or not getattr(inner, "residencies", lambda: [])():
            return error_response(409, "no_expert_cache", f"model {model!r} keeps every expert resident")
        body = await request.json()
        try:
            warmed = await asyncio.get_running_loop().run_in_executor(None, service.call, lm, lambda _m: mcp.apply(inner, body))
        except (ValueError, KeyError, TypeError) as exc:
            return error_response(400, "invalid_request", f"not a usable cache profile: {exc}")
        return {"model": model, "warmed_experts": warmed}

    @app.get("/api/v1/datasets/catalog")
    async def datasets_catalog():
        """Calibration corpora (directories written by ``mfq calibrate data`` / ``trace-data``) under the catalog's
        roots: name, path, format, sequences and tokens per split, tokenizer identity."""
        roots = list(getattr(catalog, "roots", []) or [])
        found = []
        for root in roots:
            base = Path(root)
            if not base.is_dir():
                continue
            for manifest in sorted(base.glob("**/manifest.json")):
                try:
                    doc = json.loads(manifest.read_text(encoding="utf-8"))
                except (OSError, ValueError):
                    continue
                if not str(doc.get("format", "")).startswith("mfq.calibration-corpus."):
                    continue
                found.append({"name": manifest.parent.name, "path": str(manifest.parent), "format": doc["format"],
                              "sequence_length": doc.get("sequence_length"), "domains": doc.get("domains"),
                              "tokens": doc.get("actual_tokens"), "scored_tokens": doc.get("scored_tokens"),
                              "tokenizer": doc.get("tokenizer")})
        return {"roots": roots, "datasets": found}

    @app.post("/api/v1/evaluations/probabilities")
    async def evaluation_probabilities(request: HttpRequest):
        """Log-probabilities of given continuations of a prompt under a loaded model (natural log, raw tokenization
        without special tokens).  ``mode``: ``continuation`` scores every token of each continuation, ``next_token``
        only its first.  Body: ``{"model"?, "prompt", "continuations": [...], "mode"?}``."""
        body = await request.json()
        prompt, conts, mode = body.get("prompt"), body.get("continuations"), body.get("mode", "continuation")
        if not isinstance(prompt, str) or not prompt or not isinstance(conts, list) or not 1 <= len(conts) <= 64 \
                or not all(isinstance(c, str) and c for c in conts) or mode not in ("continuation", "next_token"):
            return error_response(400, "invalid_request", "need a prompt, 1..64 non-empty continuations and mode continuation | next_token")
        try:
            lm = service.resolve(body.get("model"))
        except KeyError:
            return error_response(404, "model_not_found", f"model {body.get('model')!r} is not loaded")
        engine = lm.engine
        if engine is None or not callable(getattr(engine, "score", None)):
            return error_response(501, "probability_unavailable", "the loaded runtime does not support probability scoring")
        head = [int(t) for t in lm.tokenizer.encode(prompt)]
        tails = [[int(t) for t in lm.tokenizer.encode(c)] for c in conts]
        if not head or any(not t for t in tails):
            return error_response(400, "invalid_request", "prompt and continuations must tokenize to at least one token")

        def run(model):
            row = model.scheduler._free_row()
            if row is None:
                raise QueueFull("every batch row is busy")
            out = []
            for tail in tails:
                use = tail[:1] if mode == "next_token" else tail
                logp = engine.score(row, head + use, len(head))
                out.append({"token_ids": use, "token_logprobs": [min(0.0, float(x)) for x in logp], "log_likelihood": float(sum(logp))})
            return out

        try:
            scores = await asyncio.get_running_loop().run_in_executor(None, service.call, lm, run)
        except QueueFull as exc:
            return error_response(503, "server_busy", str(exc))
        except ValueError as exc:
            return error_response(400, "invalid_request", str(exc))
        return {"prompt_tokens": len(head), "scores": scores, "log_base": "e", "tokenization": "raw-no-special-tokens"}

    @app.get("/api/v1/runtime/sampling-profile")
    async def sampling_profile(model: str | None = None):
        """Effective sampling defaults of a loaded model and where they come from."""
        from ..formats import runtime_profile as rp
        try:
            lm = service.resolve(model)
        except KeyError:
            return error_response(404, "model_not_found", f"model {model!r} is not loaded")
        meta = getattr(lm, "meta", None) or {}
        return rp.resolve(meta.get("header_extra"), meta.get("assets"), meta.get("architecture"), meta.get("path"))

    return app
