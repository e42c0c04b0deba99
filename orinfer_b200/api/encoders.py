"""``POST /v1/embeddings`` and ``POST /v1/rerank`` (alias ``/rerank``) on the serving model.

Both run encoder passes of the loaded decoder on the engine thread, between generation steps:
an embedding is the mean-pooled, L2-normalised final hidden state; a rerank score is the
unsaturated ``yes`` minus ``no`` logit after a judgement prompt.  Request shapes, limits and
response fields follow the reference (docs/embeddings.md:19-36, docs/reranking.md:17-36,
crates/orinfer-api/src/embeddings.rs, reranking.rs:127-176); its dedicated bidirectional
encoder families (Nemotron-Embed, Qwen-Reranker) are not separate architectures here.
"""

from __future__ import annotations

import base64
import struct
from typing import Any, Dict, List

from fastapi import FastAPI
from fastapi import Request as HttpRequest
from fastapi.responses import JSONResponse

from .chat_codec import RequestError

MAX_ITEMS = 128
MAX_TOKENS = 32768


def _err(e: RequestError) -> JSONResponse:
    return JSONResponse(e.body(), status_code=e.status)


def _texts(value, what: str) -> List[str]:
    items = [value] if isinstance(value, (str, dict)) else value
    if not isinstance(items, list) or not items:
        raise RequestError(f"`{what}` must be a string or a non-empty array", param=what)
    if len(items) > MAX_ITEMS:
        raise RequestError(f"`{what}` holds more than {MAX_ITEMS} items", param=what)
    out = []
    for it in items:
        if isinstance(it, dict):
            if it.get("images"):
                raise RequestError("image inputs need a vision encoder, which this model lacks",
                                   param=what)
            it = it.get("text")
        if not isinstance(it, str):
            raise RequestError(f"`{what}` items must be strings or {{text}} objects", param=what)
        out.append(it)
    return out


def embeddings(service, body: Dict[str, Any]) -> Dict[str, Any]:
    texts = _texts(body.get("input"), "input")
    kind = body.get("input_type", "document")
    if kind not in ("document", "query"):
        raise RequestError("`input_type` must be document or query", param="input_type")
    fmt = body.get("encoding_format", "float")
    if fmt not in ("float", "base64"):
        raise RequestError("`encoding_format` must be float or base64", param="encoding_format")
    dims = body.get("dimensions")
    prefix = "query: " if kind == "query" else "passage: "
    tok = service.codec.tokenizer
    data, used = [], 0
    for i, text in enumerate(texts):
        ids = tok.encode(prefix + text)
        if len(ids) > MAX_TOKENS:
            raise RequestError(f"input {i} exceeds {MAX_TOKENS} tokens", param="input")
        vec, _ = service.worker.call(lambda eng, ids=ids: eng.encode(ids))
        if dims is not None:
            if not isinstance(dims, int) or not 1 <= dims <= vec.numel():
                raise RequestError("`dimensions` is outside 1..hidden size", param="dimensions")
            vec = vec[:dims]
            vec = vec / vec.norm().clamp_min(1e-12)       # Matryoshka truncation + renormalise
        vals = vec.tolist()
        emb = (base64.b64encode(struct.pack(f"<{len(vals)}f", *vals)).decode()
               if fmt == "base64" else vals)
        data.append({"object": "embedding", "index": i, "embedding": emb})
        used += len(ids)
    return {"object": "list", "model": service.model_name, "data": data,
            "usage": {"prompt_tokens": used, "total_tokens": used}}


def rerank(service, body: Dict[str, Any]) -> Dict[str, Any]:
    query = body.get("query")
    if not isinstance(query, str) or not query:
        raise RequestError("`query` must be a non-empty string", param="query")
    docs = _texts(body.get("documents"), "documents")
    top_n = body.get("top_n", len(docs))
    if not isinstance(top_n, int) or top_n < 1:
        raise RequestError("`top_n` must be a positive integer", param="top_n")
    instruction = body.get("instruction") or \
        "Given a query, judge whether the document answers it."
    tok = service.codec.tokenizer
    yes, no = tok.encode("yes")[-1], tok.encode("no")[-1]
    results, used = [], 0
    for i, doc in enumerate(docs):
        ids = tok.encode(f"{instruction}\nQuery: {query}\nDocument: {doc}\nAnswer (yes or no): ")
        if len(ids) > MAX_TOKENS:
            raise RequestError(f"document {i} exceeds {MAX_TOKENS} tokens", param="documents")
        _, logits = service.worker.call(lambda eng, ids=ids: eng.encode(ids))
        item = {"index": i, "relevance_score": float(logits[yes] - logits[no])}
        if body.get("return_documents"):
            item["document"] = {"text": doc}
        results.append(item)
        used += len(ids)
    results.sort(key=lambda r: (-r["relevance_score"], r["index"]))      # stable input order
    return {"model": service.model_name, "results": results[:top_n],
            "usage": {"prompt_tokens": used, "total_tokens": used}}


def install(app: FastAPI, service) -> None:
    import asyncio

    async def _run(fn, request: HttpRequest):
        try:
            body = await request.json()
            if not isinstance(body, dict):
                raise RequestError("request body must be a JSON object")
            return JSONResponse(await asyncio.get_running_loop().run_in_executor(
                None, fn, service, body))
        except RequestError as e:
            return _err(e)
        except (MemoryError, ValueError) as e:
            return _err(RequestError(str(e), status=400))

    @app.post("/v1/embeddings")
    async def _embeddings(request: HttpRequest):
        return await _run(embeddings, request)

    @app.post("/v1/rerank")
    async def _rerank(request: HttpRequest):
        return await _run(rerank, request)

    @app.post("/rerank")
    async def _rerank_alias(request: HttpRequest):
        return await _run(rerank, request)
