"""Server configuration: defaults < TOML file < OXIBONSAI_* environment < command line.

Reference: the serve crate's layered ``PartialServerConfig::merge`` (crates/oxibonsai-serve/src/config.rs, env.rs, args.rs:65-305),
its validation rules (validation.rs:3-110: port != 0, max_tokens <= 8192, temperature in [0, 2], top_p in [0, 1], bearer
token of at least 16 characters, paths must exist) and the runtime TOML sections ``[server] [sampling] [model]
[observability]`` (crates/oxibonsai-runtime/src/config.rs:13-112).
"""
from __future__ import annotations

import argparse
import os
from dataclasses import dataclass, fields, replace
from typing import Any, Mapping


@dataclass(frozen=True)
class ServerConfig:
    host: str = "0.0.0.0"
    port: int = 8080
    model_path: str | None = None
    tokenizer_path: str | None = None
    tokenizer_kind: str = "auto"
    max_tokens: int = 512
    temperature: float = 0.7
    top_k: int = 40
    top_p: float = 0.9
    repetition_penalty: float = 1.1
    seed: int = 42
    max_seq_len: int = 4096
    max_input_tokens: int = 32768
    max_concurrent: int = 64
    request_timeout_ms: int = 120000
    bearer_token: str | None = None
    log_level: str = "info"
    json_logs: bool = False
    metrics_enabled: bool = True
    metrics_path: str = "/metrics"
    quantization_hint: str | None = None
    kv_cache: str = "f16"
    tensor_parallel: int = 1          # > 1: launch with torchrun, one process per GPU; rank 0 serves HTTP, the others follow its commands
    tp_elastic: bool = False          # with tensor_parallel > 1: watch the ranks' heartbeats and re-form the group at a smaller degree when one is lost
    tp_heartbeat_timeout: float = 5.0 # seconds without a heartbeat after which a rank counts as lost
    replicas: int = 1                 # > 1: one engine + scheduler per GPU (cuda:0 .. cuda:N-1) in this process, requests routed between them
    prefill_chunk_tokens: int = 512   # prompt tokens prefilled between two decode steps of the running streams
    prefill_chunk_boost: int = 4      # chunks this many times as long while fewer than a quarter of the slots decode
    admit_tokens_per_step: int = 512  # queued prompts admitted before one decode step while they cost no more than this many prompt tokens (a prompt
                                      # counts for at least 128); 0: one prompt chunk per step.  Fills the batch on short generations.
    kv_policy: str = "off"            # off | adaptive | aggressive: admit new sequences with Q8 / Q4 KV pages under memory pressure
    queue_capacity: int = 1024
    chat_template: str = "auto"       # chatml | qwen | llama3 | mistral | gemma, or auto: inferred from the model's name, ChatML otherwise
    overlap_steps: bool = False       # launch decode step k + 1 before the tokens of step k are delivered (single-process engines)
    native_front: bool = True         # C++ HTTP / SSE front (sockets, parsing, token streaming); off: uvicorn

    def validate(self, check_paths: bool = True) -> "ServerConfig":
        errs = []
        if not 0 < self.port < 65536:
            errs.append("port must be in 1..65535")
        if not 0 < self.max_tokens <= 8192:
            errs.append("max_tokens must be in 1..8192")
        if not 0.0 <= self.temperature <= 2.0:
            errs.append("temperature must be in [0, 2]")
        if not 0.0 <= self.top_p <= 1.0:
            errs.append("top_p must be in [0, 1]")
        if self.bearer_token is not None and len(self.bearer_token) < 16:
            errs.append("bearer_token must have at least 16 characters")
        if self.max_concurrent < 1:
            errs.append("max_concurrent must be positive")
        if self.tensor_parallel < 1 or self.replicas < 1:
            errs.append("tensor_parallel and replicas must be positive")
        if self.tensor_parallel > 1 and self.replicas > 1:
            errs.append("tensor_parallel and replicas cannot be combined in one server")
        if self.admit_tokens_per_step < 0 or self.prefill_chunk_tokens < 1 or self.prefill_chunk_boost < 1 or self.queue_capacity < 1:
            errs.append("prefill_chunk_tokens, prefill_chunk_boost and queue_capacity must be >= 1, admit_tokens_per_step >= 0")
        if self.kv_policy not in ("off", "adaptive", "aggressive"):
            errs.append("kv_policy must be one of off, adaptive, aggressive")
        if self.chat_template not in ("auto", "chatml", "qwen", "llama3", "mistral", "gemma"):
            errs.append("chat_template must be one of auto, chatml, qwen, llama3, mistral, gemma")
        if self.kv_cache.lower() not in ("f32", "f16", "q8", "q4"):
            errs.append("kv_cache must be one of f32, f16, q8, q4")
        if check_paths:
            for name in ("model_path", "tokenizer_path"):
                p = getattr(self, name)
                if p is not None and not os.path.exists(p):
                    errs.append(f"{name} does not exist: {p}")
        if errs:
            raise ValueError("invalid server configuration: " + "; ".join(errs))
        return self


_TOML_MAP = {
    ("server", "host"): "host", ("server", "port"): "port", ("server", "max_concurrent"): "max_concurrent",
    ("server", "request_timeout_ms"): "request_timeout_ms", ("server", "bearer_token"): "bearer_token",
    ("sampling", "temperature"): "temperature", ("sampling", "top_k"): "top_k", ("sampling", "top_p"): "top_p",
    ("sampling", "repetition_penalty"): "repetition_penalty", ("sampling", "max_tokens"): "max_tokens", ("sampling", "seed"): "seed",
    ("model", "model_path"): "model_path", ("model", "tokenizer_path"): "tokenizer_path", ("model", "max_seq_len"): "max_seq_len",
    ("model", "kv_cache"): "kv_cache", ("model", "tensor_parallel"): "tensor_parallel", ("model", "replicas"): "replicas", ("model", "tp_elastic"): "tp_elastic", ("model", "tp_heartbeat_timeout"): "tp_heartbeat_timeout", ("model", "kv_policy"): "kv_policy",
    ("server", "native_front"): "native_front", ("model", "chat_template"): "chat_template", ("server", "overlap_steps"): "overlap_steps", ("server", "prefill_chunk_tokens"): "prefill_chunk_tokens", ("server", "prefill_chunk_boost"): "prefill_chunk_boost", ("server", "admit_tokens_per_step"): "admit_tokens_per_step",
    ("observability", "log_level"): "log_level", ("observability", "json_logs"): "json_logs",
    ("observability", "metrics_enabled"): "metrics_enabled", ("observability", "metrics_path"): "metrics_path",
}


def _coerce(field_type: Any, value: Any) -> Any:
    t = str(field_type)
    if value is None:
        return None
    if "bool" in t:
        return value if isinstance(value, bool) else str(value).strip().lower() in ("1", "true", "yes", "on")
    if "int" in t:
        return int(value)
    if "float" in t:
        return float(value)
    return str(value)


def from_toml(path: str) -> dict:
    import tomllib
    with open(path, "rb") as f:
        doc = tomllib.load(f)
    out = {}
    for (sec, key), name in _TOML_MAP.items():
        if sec in doc and key in doc[sec]:
            out[name] = doc[sec][key]
    # flat keys at the top level are accepted as well
    names = {f.name for f in fields(ServerConfig)}
    out.update({k: v for k, v in doc.items() if k in names and not isinstance(v, dict)})
    return out


def from_env(env: Mapping[str, str] | None = None) -> dict:
    env = os.environ if env is None else env
    out = {}
    for f in fields(ServerConfig):
        v = env.get("OXIBONSAI_" + f.name.upper())
        if v is not None and v != "":
            out[f.name] = v
    return out


def build_arg_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="oxibonsai-serve", description="OpenAI-compatible server for sub-2-bit Qwen3 checkpoints on B200")
    ap.add_argument("--config", help="TOML configuration file")
    for f in fields(ServerConfig):
        flag = "--" + f.name.replace("_", "-")
        if "bool" in str(f.type):
            ap.add_argument(flag, dest=f.name, default=None, action=argparse.BooleanOptionalAction)
        else:
            ap.add_argument(flag, dest=f.name, default=None)
    return ap


def load_config(argv: list[str] | None = None, env: Mapping[str, str] | None = None, check_paths: bool = True) -> ServerConfig:
    args = vars(build_arg_parser().parse_args(argv or []))
    layers: list[dict] = []
    if args.get("config"):
        layers.append(from_toml(args["config"]))
    layers.append(from_env(env))
    layers.append({k: v for k, v in args.items() if k != "config" and v is not None})
    cfg = ServerConfig()
    types = {f.name: f.type for f in fields(ServerConfig)}
    for layer in layers:
        cfg = replace(cfg, **{k: _coerce(types[k], v) for k, v in layer.items() if k in types})
    return cfg.validate(check_paths)
