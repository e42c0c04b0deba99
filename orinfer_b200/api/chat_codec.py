"""Chat request decoding: validation, defaults, template rendering, tokenisation.

Behavioural contract follows the reference's codec
(crates/orinfer-api/src/server/chat.rs:97-142 request fields with unknown fields
rejected, :341-830 prepare; crates/orinfer-api/src/server/defaults.rs:23-110 defaults
merging: request > deployment > model, explicit null clears a deployment default,
grouped fields override as a group).
"""

from __future__ import annotations

import json
import os
import secrets
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Dict, List, Optional, Sequence, Tuple

import jinja2

from ..core.sampling import SamplingOptions

MAX_STOPS = 4
MAX_TOOLS = 128


class RequestError(ValueError):
    """A client error: becomes an OpenAI-style error body."""

    def __init__(self, message: str, param: Optional[str] = None, code: Optional[str] = None,
                 status: int = 400, err_type: str = "invalid_request_error"):
        super().__init__(message)
        self.message, self.param, self.code, self.status, self.type = \
            message, param, code, status, err_type

    def body(self) -> dict:
        return {"error": {"message": self.message, "type": self.type, "param": self.param,
                          "code": self.code}}


# --------------------------------------------------------------------------- tokenizers
class ByteTokenizer:
    """Fallback for random-init models without tokenizer assets: UTF-8 bytes are ids
    0..255, followed by the control tokens."""

    SPECIALS = ["<|endoftext|>", "<|im_start|>", "<|im_end|>", "<think>", "</think>",
                "<tool_call>", "</tool_call>", "<|vision_start|>", "<|image_pad|>",
                "<|vision_end|>", "<|audio_start|>", "<|audio_pad|>", "<|audio_end|>"]

    def __init__(self, vocab: int):
        if vocab < 256 + len(self.SPECIALS):
            raise ValueError("vocabulary too small for the byte tokenizer")
        self.vocab = vocab
        self.special_ids = {s: 256 + i for i, s in enumerate(self.SPECIALS)}
        self.eos_ids = (self.special_ids["<|im_end|>"], self.special_ids["<|endoftext|>"])

    def encode(self, text: str) -> List[int]:
        out: List[int] = []
        i = 0
        while i < len(text):
            hit = next((s for s in self.SPECIALS if text.startswith(s, i)), None)
            if hit:
                out.append(self.special_ids[hit])
                i += len(hit)
            else:
                out.extend(text[i].encode("utf-8"))
                i += 1
        return out

    def encode_plain(self, text: str) -> List[int]:
        """Bytes only: control-token spellings in the text stay ordinary characters."""
        return list(text.encode("utf-8"))

    def token_bytes(self, tok: int) -> bytes:
        if tok < 256:
            return bytes([tok])
        idx = tok - 256
        return self.SPECIALS[idx].encode() if idx < len(self.SPECIALS) else b""

    def decode(self, ids: Sequence[int]) -> str:
        return b"".join(self.token_bytes(t) for t in ids).decode("utf-8", errors="replace")

    def token_id(self, text: str) -> Optional[int]:
        return self.special_ids.get(text)


class HFTokenizer:
    """``tokenizer.json`` through the ``tokenizers`` library."""

    def __init__(self, path: Path, eos: Sequence[int] = ()):
        from tokenizers import Tokenizer
        self.tk = Tokenizer.from_file(str(path))
        self.vocab = self.tk.get_vocab_size()
        self.eos_ids = tuple(eos)

    def encode(self, text: str) -> List[int]:
        return self.tk.encode(text, add_special_tokens=False).ids

    def decode(self, ids: Sequence[int]) -> str:
        return self.tk.decode(list(ids), skip_special_tokens=False)

    def token_bytes(self, tok: int) -> bytes:
        return self.decode([tok]).encode("utf-8")

    def token_id(self, text: str) -> Optional[int]:
        return self.tk.token_to_id(text)


DEFAULT_TEMPLATE = (
    "{%- if tools -%}<|im_start|>system{{ '\\n' }}# Tools{{ '\\n' }}{{ tools | tojson }}"
    "<|im_end|>{{ '\\n' }}{%- endif -%}"
    "{%- for m in messages -%}<|im_start|>{{ m.role }}{{ '\\n' }}"
    "{%- if m.content is string -%}{{ m.content }}{%- elif m.content -%}"
    "{%- for part in m.content -%}{%- if part.type == 'text' -%}{{ part.text }}{%- endif -%}"
    "{%- endfor -%}{%- endif -%}"
    "{%- if m.tool_calls -%}{%- for c in m.tool_calls -%}{{ '\\n' }}<tool_call>{{ '\\n' }}"
    "{{ {'name': c.function.name, 'arguments': c.function.arguments} | tojson }}"
    "{{ '\\n' }}</tool_call>{%- endfor -%}{%- endif -%}<|im_end|>{{ '\\n' }}{%- endfor -%}"
    "{%- if add_generation_prompt -%}<|im_start|>assistant{{ '\\n' }}"
    "{%- if enable_thinking -%}<think>{{ '\\n' }}{%- endif -%}{%- endif -%}")


def _tojson(value, indent=None):
    # Python's default separators, as chat templates written for transformers expect
    return json.dumps(value, ensure_ascii=False, indent=indent)


# --------------------------------------------------------------------------- request model
ALLOWED_FIELDS = {
    "model", "messages", "temperature", "top_p", "top_k", "n", "stream", "stream_options",
    "stop", "max_tokens", "max_completion_tokens", "presence_penalty", "frequency_penalty",
    "repetition_penalty", "logit_bias", "logprobs", "top_logprobs", "seed", "user", "tools",
    "tool_choice", "parallel_tool_calls", "response_format", "enable_thinking",
    "chat_template_kwargs", "reasoning_effort", "thinking_token_budget", "prompt_cache_key",
    "prompt_cache_retention", "ignore_eos", "image_processing", "store", "metadata",
    "min_tokens", "cache_prompt", "service_tier",
    # "clamp": an output limit that does not fit the context is shortened instead of refused
    # (what the Ollama routes ask for: `num_predict` is a wish there, not a contract)
    "output_limit",
}



THINKING_FIELDS = ("enable_thinking", "thinking", "reasoning_effort")     # in template kwargs
BUDGET_FIELDS = ("thinking_budget", "thinking_token_budget")


def merge_defaults(request: Dict[str, Any], deployment: Dict[str, Any]) -> Dict[str, Any]:
    """request > deployment.  A field the request names (even as ``false``, ``[]`` or
    ``null``) is the request's; ``null`` then means "not set".  Related controls override as
    one group, so a default can neither contradict nor defeat the spelling the client chose:
    the two output limits; the thinking switches (top level or inside
    ``chat_template_kwargs``); the two spellings of the thinking budget.  ``stream`` off takes
    a default ``stream_options`` with it and ``logprobs`` off a default ``top_logprobs``.
    ``chat_template_kwargs`` merge key by key (crates/orinfer-api/src/server/defaults.rs:40-104)."""
    kwargs = request.get("chat_template_kwargs")
    kwargs = kwargs if isinstance(kwargs, dict) else {}
    output_override = "max_tokens" in request or "max_completion_tokens" in request
    thinking_override = ("enable_thinking" in request or "reasoning_effort" in request
                         or any(k in kwargs for k in THINKING_FIELDS))
    budget_override = ("thinking_token_budget" in request
                       or any(k in kwargs for k in BUDGET_FIELDS))
    stream_off = "stream" in request and not request["stream"]
    logprobs_off = "logprobs" in request and not request["logprobs"]
    out = dict(request)
    for name, value in deployment.items():
        if name == "chat_template_kwargs" and isinstance(value, dict):
            if "chat_template_kwargs" in request and not isinstance(
                    request["chat_template_kwargs"], dict):
                continue                              # an explicit null clears the whole map
            merged = dict(kwargs)
            for key, v in value.items():
                if thinking_override and key in THINKING_FIELDS \
                        or budget_override and key in BUDGET_FIELDS:
                    continue
                merged.setdefault(key, v)
            out["chat_template_kwargs"] = merged
            continue
        if (name in request
                or output_override and name in ("max_tokens", "max_completion_tokens")
                or thinking_override and name in ("enable_thinking", "reasoning_effort")
                or budget_override and name == "thinking_token_budget"
                or stream_off and name == "stream_options"
                or logprobs_off and name == "top_logprobs"):
            continue
        out[name] = value
    return {k: v for k, v in out.items() if v is not None}


def thinking_budget_of(req: Dict[str, Any]) -> Optional[int]:
    """The thinking budget a request asks for: the top-level field wins over the template
    variables; the two spellings inside ``chat_template_kwargs`` may not disagree; a budget is
    a non-negative integer (not a boolean, a fraction or a string)."""
    kwargs = req.get("chat_template_kwargs") or {}
    inner = [kwargs[k] for k in BUDGET_FIELDS if k in kwargs and kwargs[k] is not None]
    for value, where in [(req.get("thinking_token_budget"), "thinking_token_budget")] + \
            [(v, "chat_template_kwargs.thinking_budget") for v in inner]:
        if value is not None and (isinstance(value, bool) or not isinstance(value, int)
                                  or value < 0):
            raise RequestError("a thinking budget is a non-negative integer",
                               param="thinking_token_budget" if "." not in where else where)
    if len(inner) == 2 and inner[0] != inner[1]:
        raise RequestError("`thinking_budget` and `thinking_token_budget` disagree",
                           param="chat_template_kwargs.thinking_budget")
    if req.get("thinking_token_budget") is not None:
        return req["thinking_token_budget"]
    return inner[0] if inner else None


@dataclass
class ModelDefaults:
    thinking: bool = False
    temperature: float = 0.0
    top_p: float = 1.0
    top_k: int = 0
    presence_penalty: float = 0.0
    max_tokens: int = 1024
    frequency_penalty: float = 0.0
    repetition_penalty: float = 1.0

    @classmethod
    def from_generation_config(cls, gen: Dict[str, Any]) -> "ModelDefaults":
        """Sampling defaults a checkpoint ships in ``generation_config.json`` (the model
        card's recommendation); requests and deployment defaults are applied on top
        (crates/orinfer-api/src/server/chat/generation_defaults.rs:41-60).  ``do_sample:
        false`` means greedy whatever temperature is written beside it."""
        d = cls()
        number = lambda key, old: float(gen[key]) if isinstance(gen.get(key), (int, float)) \
            and not isinstance(gen.get(key), bool) else old
        if gen.get("do_sample") is not False:
            d.temperature = number("temperature", d.temperature)
        d.top_p = number("top_p", d.top_p)
        top_k = gen.get("top_k")
        if isinstance(top_k, int) and not isinstance(top_k, bool):
            d.top_k = 0 if top_k < 0 else top_k
        d.presence_penalty = number("presence_penalty", d.presence_penalty)
        d.frequency_penalty = number("frequency_penalty", d.frequency_penalty)
        d.repetition_penalty = number("repetition_penalty", d.repetition_penalty)
        return d


@dataclass
class Prepared:
    """A validated request ready for the engine."""
    prompt_ids: List[int]
    sampling: SamplingOptions
    max_new: int
    stream: bool
    include_usage: bool
    stop_ids: Tuple[int, ...]
    stop_strings: List[str]
    ignore_eos: bool
    want_logprobs: bool
    thinking: bool
    thinking_budget: Optional[int]
    json_schema: Optional[dict]
    json_object: bool
    tools: List[dict]
    tool_choice: Any
    parallel_tool_calls: bool
    model: str
    prompt_text: str = ""
    cache_prompt: bool = True
    images: Optional[Any] = None      # api.images.BoundImages when the prompt holds images
    audio: Optional[Any] = None       # api.audio.BoundAudio of a transcription request
    token_events: bool = False        # completions route: report every committed token id


class ChatCodec:
    def __init__(self, tokenizer, template: Optional[str] = None,
                 defaults: Optional[ModelDefaults] = None, context: int = 32768,
                 model_name: str = "orinfer", protect_controls: bool = True):
        self.tokenizer = tokenizer
        self.env = jinja2.Environment(trim_blocks=False, lstrip_blocks=False,
                                      extensions=["jinja2.ext.loopcontrols"])
        self.env.filters["tojson"] = _tojson

        def raise_exception(message):          # templates written for transformers call this
            raise jinja2.TemplateError(message)
        self.env.globals["raise_exception"] = raise_exception
        # control tokens may come only from the template source or the server (token_boundary.py)
        self.boundary = None
        if protect_controls:
            from .token_boundary import Boundary, BoundaryError
            try:
                self.boundary = Boundary(tokenizer)
            except BoundaryError:
                self.boundary = None
        source = template or DEFAULT_TEMPLATE
        self.template = self.env.from_string(
            self.boundary.template(source) if self.boundary else source)
        self.defaults = defaults or ModelDefaults()
        self.context = context
        self.model_name = model_name
        self.images = None            # api.images.ImageFrontend of a vision-capable model
        self.tool_format = "xml"      # "dsml": DeepSeek-style call blocks (api/dsml.py)
        # an explicit output limit that does not fit the context is refused, not shortened
        self.strict_context = True

    @classmethod
    def load(cls, model_dir: Path, vocab: int, context: int, model_name: str) -> "ChatCodec":
        model_dir = Path(model_dir)
        template = None
        tpl = model_dir / "chat_template.jinja"
        if tpl.exists():
            template = tpl.read_text()
        elif (model_dir / "tokenizer_config.json").exists():
            # older checkpoints keep the template inside the tokenizer configuration
            held = json.loads((model_dir / "tokenizer_config.json").read_text()).get("chat_template")
            if isinstance(held, str) and held.strip():
                template = held
        eos: List[int] = []
        defaults = None
        gen = model_dir / "generation_config.json"
        if gen.exists():
            held = json.loads(gen.read_text())
            e = held.get("eos_token_id", [])
            eos = [e] if isinstance(e, int) else list(e or [])
            defaults = ModelDefaults.from_generation_config(held)
        tok_file = model_dir / "tokenizer.json"
        tokenizer = HFTokenizer(tok_file, eos) if tok_file.exists() else ByteTokenizer(vocab)
        if tokenizer.vocab > vocab:
            raise ValueError("tokenizer vocabulary exceeds the model vocabulary")
        return cls(tokenizer, template, defaults, context, model_name)

    # ----------------------------------------------------------------- validation
    def prepare(self, body: Dict[str, Any], deployment_defaults: Optional[dict] = None) -> Prepared:
        if not isinstance(body, dict):
            raise RequestError("request body must be a JSON object")
        unknown = sorted(set(body) - ALLOWED_FIELDS)
        if unknown:
            raise RequestError(f"unknown field `{unknown[0]}`", param=unknown[0])
        req = merge_defaults(body, deployment_defaults or {})
        from .messages import MessageError, normalize
        try:
            # one shape for every wire form: text parts joined, ``null`` content empty, tool
            # call arguments parsed, developer folded into system, calls answered
            messages = normalize(req.get("messages"), self.tool_format)
        except MessageError as e:
            raise RequestError(str(e), param=e.param)
        for name in ("stream", "logprobs", "enable_thinking", "ignore_eos", "store",
                     "parallel_tool_calls", "cache_prompt"):
            if req.get(name) is not None and not isinstance(req[name], bool):
                raise RequestError(f"`{name}` must be true, false or null", param=name)
        if body.get("max_tokens") is not None and body.get("max_completion_tokens") is not None:
            raise RequestError("specify only one output-token limit",
                               param="max_completion_tokens")
        if req.get("reasoning_effort") is not None and req["reasoning_effort"] not in EFFORTS:
            raise RequestError("`reasoning_effort` is one of " + "/".join(EFFORTS),
                               param="reasoning_effort")
        if req.get("reasoning_effort") == "none" and req.get("enable_thinking") is True:
            raise RequestError("`enable_thinking` conflicts with reasoning_effort=none",
                               param="enable_thinking")
        key = req.get("prompt_cache_key")
        if key is not None and (not isinstance(key, str) or not 1 <= len(key) <= 64):
            raise RequestError("`prompt_cache_key` takes 1 to 64 characters",
                               param="prompt_cache_key")
        if req.get("prompt_cache_retention") not in (None, "in-memory", "24h"):
            raise RequestError("`prompt_cache_retention` is in-memory or 24h",
                               param="prompt_cache_retention")
        if req.get("n", 1) != 1:
            raise RequestError("only n = 1 is supported", param="n")
        if req.get("store") is True:
            raise RequestError("`store` is not supported", param="store")
        meta = req.get("metadata")
        if meta is not None and (not isinstance(meta, dict) or len(meta) > 16):
            raise RequestError("`metadata` accepts at most 16 string pairs", param="metadata")
        tools = req.get("tools") or []
        if len(tools) > MAX_TOOLS:
            raise RequestError(f"at most {MAX_TOOLS} tools", param="tools")
        stop = req.get("stop")
        stops = [stop] if isinstance(stop, str) else list(stop or [])
        if len(stops) > MAX_STOPS or any(not isinstance(s, str) or not s for s in stops):
            raise RequestError(f"`stop` accepts up to {MAX_STOPS} non-empty strings", param="stop")

        kwargs = dict(req.get("chat_template_kwargs") or {})
        effort = req.get("reasoning_effort", kwargs.get("reasoning_effort"))
        thinking = req.get("enable_thinking", kwargs.get("enable_thinking",
                                                         kwargs.get("thinking")))
        if thinking is None:
            thinking = (effort not in (None, "none")) if effort is not None \
                else self.defaults.thinking
        budget = thinking_budget_of(req)

        d = self.defaults
        seed = req.get("seed")
        if seed is None:
            seed = secrets.randbits(64)
        elif not isinstance(seed, int) or not -2 ** 63 <= seed < 2 ** 64:
            raise RequestError("`seed` must be a 64-bit integer", param="seed")
        top_k = req.get("top_k", d.top_k)
        if top_k in (-1, None):
            top_k = 0
        bias_in = req.get("logit_bias") or {}
        try:
            bias = {int(k): float(v) for k, v in bias_in.items()}
        except (TypeError, ValueError, AttributeError):
            raise RequestError("`logit_bias` maps token ids to numbers", param="logit_bias")
        vocab = getattr(self.tokenizer, "vocab", None)
        for tok in bias:
            if tok < 0 or (vocab is not None and tok >= vocab):
                raise RequestError(f"token {tok} is not in the vocabulary",
                                   param=f"logit_bias.{tok}")
        want_lp = bool(req.get("logprobs", False))
        top_lp = req.get("top_logprobs")
        if top_lp is not None and not want_lp:
            raise RequestError("`top_logprobs` requires `logprobs`", param="top_logprobs")
        sampling = SamplingOptions(
            temperature=float(req.get("temperature", d.temperature)),
            top_p=float(req.get("top_p", d.top_p)), top_k=int(top_k),
            presence_penalty=float(req.get("presence_penalty", d.presence_penalty)),
            frequency_penalty=float(req.get("frequency_penalty", d.frequency_penalty)),
            repetition_penalty=float(req.get("repetition_penalty", d.repetition_penalty)),
            seed=seed & (2 ** 64 - 1), logit_bias=bias,
            top_logprobs=(top_lp if top_lp is not None else (0 if want_lp else None)))
        try:
            sampling.validate()
        except ValueError as e:
            name = str(e).split(":")[0]
            raise RequestError(str(e), param=name)

        rf = req.get("response_format") or {"type": "text"}
        schema, json_object = None, False
        if rf.get("type") == "json_schema":
            js = rf.get("json_schema") or {}
            schema = js.get("schema")
            if not isinstance(schema, (dict, bool)):
                raise RequestError("`json_schema.schema` must be an object",
                                   param="response_format.json_schema.schema")
            _check_schema(schema)
        elif rf.get("type") == "json_object":
            json_object = True
        elif rf.get("type") != "text":
            raise RequestError("unknown response_format type", param="response_format")
        constrained = schema is not None or json_object
        if constrained and stops:
            raise RequestError("`stop` cannot be combined with a constrained response",
                               param="stop")

        if self.boundary is not None:
            messages = self.boundary.escape_value(messages)
            tools = self.boundary.escape_value(tools)
            kwargs = self.boundary.escape_value(kwargs)
        if self.tool_format == "dsml":
            # results follow their calls' order; past calls are shown in wire syntax
            from . import dsml
            mark = dsml.MARK
            if self.boundary is not None and mark in self.boundary.tokens:
                mark = self.boundary.control(mark)
            messages = dsml.reorder_tool_results(messages)
            messages = [dict(m, content=((m.get("content") or "") + "\n\n" +
                                         dsml.render_calls(m["tool_calls"], mark)).lstrip("\n"),
                             tool_calls=None)
                        if m.get("role") == "assistant" and m.get("tool_calls") else m
                        for m in messages]
        bound = None
        has_images = any(isinstance(m.get("content"), list) and any(
            isinstance(p, dict) and p.get("type") == "image_url" for p in m["content"])
            for m in messages)
        if has_images and self.images is None:
            raise RequestError("this model takes no image inputs", param="messages")
        if self.images is not None:
            from .images import ImageOptions
            opts = ImageOptions.parse(req.get("image_processing"))
            decoded = []
            if has_images:
                messages, decoded = self.images.extract(
                    messages, opts, self.boundary.controls if self.boundary else None)
        text = self.render(messages, tools, bool(thinking), kwargs)
        ids = self.encode_rendered(text)
        text = self.display(text)
        if self.images is not None:
            bound = self.images.bind(ids, decoded, opts)
            ids = bound.prompt_ids
            bound = bound if bound.images else None
        limit = req.get("max_completion_tokens")
        limit_name = "max_completion_tokens" if limit is not None else "max_tokens"
        if limit is None:
            limit = req.get("max_tokens")
        # explicit: the client itself named a limit (deployment defaults are shortened to fit)
        explicit = (body.get("max_completion_tokens") is not None
                    or body.get("max_tokens") is not None) \
            and req.get("output_limit", "strict") != "clamp"
        max_new = limit if limit is not None else d.max_tokens
        if not isinstance(max_new, int) or isinstance(max_new, bool) or max_new < 1:
            raise RequestError(f"`{limit_name}` must be a positive integer", param=limit_name)
        if len(ids) >= self.context:
            raise RequestError(
                f"the prompt of {len(ids)} tokens exceeds the context window of "
                f"{self.context} tokens", param="messages", code="context_length_exceeded")
        if explicit and len(ids) + max_new > self.context and self.strict_context:
            # a limit the client asked for is kept or refused, never silently shortened
            raise RequestError(
                f"the request exceeds the context window of {self.context} tokens: "
                f"{len(ids)} prompt tokens + {max_new} output tokens", param=limit_name,
                code="context_length_exceeded")
        max_new = min(max_new, self.context - len(ids))
        if thinking and budget is not None and max_new < 2:
            raise RequestError("a thinking budget needs room for the end of thinking and an "
                               "answer token", param=limit_name)
        stream_opts = req.get("stream_options") or {}
        if not isinstance(stream_opts, dict):
            raise RequestError("`stream_options` must be an object", param="stream_options")
        if stream_opts.get("include_obfuscation"):
            raise RequestError("only false is supported",
                               param="stream_options.include_obfuscation")
        return Prepared(
            prompt_ids=ids, sampling=sampling, max_new=max_new, stream=bool(req.get("stream")),
            include_usage=bool(stream_opts.get("include_usage")),
            stop_ids=tuple(self.tokenizer.eos_ids), stop_strings=stops,
            ignore_eos=bool(req.get("ignore_eos", False)), want_logprobs=want_lp,
            thinking=bool(thinking), thinking_budget=budget, json_schema=schema,
            json_object=json_object, tools=tools, tool_choice=req.get("tool_choice", "auto"),
            parallel_tool_calls=bool(req.get("parallel_tool_calls", True)),
            model=req.get("model") or self.model_name, prompt_text=text,
            cache_prompt=bool(req.get("cache_prompt", True)), images=bound)

    def encode_rendered(self, text: str) -> List[int]:
        return self.boundary.encode(text) if self.boundary else self.tokenizer.encode(text)

    def display(self, text: str) -> str:
        """Rendered text with the private handles shown as their control-token spellings."""
        if self.boundary is None:
            return text
        names = {str(i): s for s, i in self.boundary.tokens.items()}
        return self.boundary._split.sub(
            lambda m: self.boundary.prefix if m.group(1) == "p" else names.get(m.group(1), ""),
            text)

    def render(self, messages, tools, thinking: bool, kwargs: Optional[dict] = None) -> str:
        ctx = dict(kwargs or {})
        ctx.update(messages=messages, tools=tools or None, add_generation_prompt=True,
                   enable_thinking=thinking)
        try:
            return self.template.render(**ctx)
        except jinja2.TemplateError as e:
            raise RequestError(f"chat template failed: {e}", param="messages")


def validate_defaults(codec: "ChatCodec", defaults: Dict[str, Any]) -> None:
    """Deployment defaults are checked when the service starts, not when the first request
    trips over them: they may not name what only a client can (`model`, `messages`), and the
    request they make with a one-line conversation must itself be valid
    (crates/orinfer-api/src/server/defaults.rs:6-21)."""
    if not isinstance(defaults, dict):
        raise ValueError("default_request_params must be a JSON object")
    for name in ("model", "messages"):
        if name in defaults:
            raise ValueError(f"default_request_params.{name}: must be supplied by the client")
    unknown = sorted(set(defaults) - ALLOWED_FIELDS)
    if unknown:
        raise ValueError(f"default_request_params.{unknown[0]}: unknown field")
    if not defaults:
        return
    try:
        codec.prepare({"messages": [{"role": "user", "content": "Hello"}]}, defaults)
    except RequestError as e:
        where = f".{e.param}" if e.param else ""
        raise ValueError(f"default_request_params{where}: {e.message}") from e


EFFORTS = ("none", "minimal", "low", "medium", "high", "xhigh", "max")
SCHEMA_PARAM = "response_format.json_schema.schema"


def _check_schema(schema, depth: int = 0, limit: int = 64, param: str = SCHEMA_PARAM) -> None:
    """What the constraint compiler will not be given: schemas nested deeper than ``limit``,
    references that leave the document, vendor extensions, malformed containers."""
    if depth > limit:
        raise RequestError("JSON schema nests too deeply", param=param)
    if isinstance(schema, bool):
        return
    if not isinstance(schema, dict):
        raise RequestError("a JSON schema is an object or a boolean", param=param)
    ref = schema.get("$ref")
    if isinstance(ref, str) and not ref.startswith("#"):
        raise RequestError("only local schema references are supported", param=param)
    if "x-guidance" in schema:
        raise RequestError("x-guidance schema extensions are not supported", param=param)
    for key in ("properties", "$defs", "definitions", "patternProperties"):
        if key in schema:
            if not isinstance(schema[key], dict):
                raise RequestError(f"schema `{key}` must be an object", param=param)
            for child in schema[key].values():
                _check_schema(child, depth + 1, limit, param)
    for key in ("items", "additionalProperties", "not", "if", "then", "else"):
        if key in schema:
            _check_schema(schema[key], depth + 1, limit, param)
    for key in ("anyOf", "allOf", "oneOf", "prefixItems"):
        if key in schema:
            if not isinstance(schema[key], list):
                raise RequestError(f"schema `{key}` must be an array", param=param)
            for child in schema[key]:
                _check_schema(child, depth + 1, limit, param)

