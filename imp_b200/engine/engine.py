"""The Python entry point: a thin layer over the C API (include/imp_b200/imp.h).

In the reference's manner (include/imp/imp.h:34-143): a model handle, a
context with engine settings, `generate` for whole requests, and the token
level pair prefill / decode-step, here as `submit` + `step`.  Requests are
lists of token ids (this engine has no tokenizer).  Everything that happens
(loading, scheduling, the step function, sampling) happens in the library;
this module converts arguments and results.

    from imp_b200 import Engine, EngineConfig, GenerateParams
    eng = Engine.from_folder("model_dir", EngineConfig(compute_dtype="bfloat16"))
    outs = eng.generate([[1, 2, 3]], GenerateParams(max_tokens=16, temperature=0.0))
"""
from __future__ import annotations

import ctypes
import enum
import json
from dataclasses import dataclass, field
from typing import Any, Dict, Hashable, List, Optional, Sequence

from .. import capi
from ..config.engine_config import EngineConfig
from ..config.model_config import ModelConfig


class RequestStatus(enum.Enum):
    WAITING = 0
    RUNNING = 1
    FINISHED = 2
    CANCELLED = 3
    OUT_OF_MEMORY = 4


class FinishReason(enum.Enum):
    NONE = 0
    EOS = 1
    LENGTH = 2          # max_tokens reached
    CONTEXT = 3         # the sequence reached max_seq_len


@dataclass
class GenerateParams:
    """Per-request generation settings; fields and defaults of the reference's
    ImpGenerateParams (include/imp/imp.h:61-85, src/api/imp_api.cpp:76-102) that apply here."""

    temperature: float = 0.7
    top_p: float = 0.9
    top_k: int = 40
    max_tokens: int = 256
    seed: int = -1
    min_p: float = 0.0
    repetition_penalty: float = 1.0
    frequency_penalty: float = 0.0
    presence_penalty: float = 0.0
    repeat_last_n: int = 0
    typical_p: float = 1.0
    dry_multiplier: float = 0.0
    dry_base: float = 1.75
    dry_allowed_length: int = 2
    dry_penalty_last_n: int = 0
    mirostat: int = 0
    mirostat_tau: float = 5.0
    mirostat_eta: float = 0.1
    ignore_eos: bool = False

    def to_c(self) -> "capi.ImpGenerateParams":
        p = capi.ImpGenerateParams()
        for name, _ in capi.ImpGenerateParams._fields_:
            setattr(p, name, int(getattr(self, name)) if name in ("ignore_eos", "seed") else getattr(self, name))
        return p


@dataclass
class StepEntry:
    """The next tokens of one request, and which of them should yield logits."""

    rid: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = field(default_factory=list)   # indices into `tokens`


@dataclass
class StepOutput:
    rid: int
    token: int
    finished: bool
    status: RequestStatus
    finish_reason: FinishReason = FinishReason.NONE


class Request:
    """Handle of a submitted request: its state is read from the engine when asked for."""

    def __init__(self, engine: "Engine", rid: int, prompt: Sequence[int], refused: bool = False):
        self._engine, self.rid, self.prompt = engine, rid, list(prompt)
        self._refused = refused
        self._final: Optional[Dict[str, Any]] = None

    def _info(self) -> Dict[str, Any]:
        if self._final is not None:
            return self._final
        if self._refused:
            return {"status": RequestStatus.OUT_OF_MEMORY, "finish_reason": FinishReason.NONE, "n_output": 0,
                    "n_computed": 0, "n_preempted": 0, "output": []}
        lib, ctx = capi.load(), self._engine._ctx
        info = capi.ImpRequestInfo()
        capi.check(lib.imp_request_info(ctx, self.rid, ctypes.byref(info)))
        out = {"status": RequestStatus(info.status), "finish_reason": FinishReason(info.finish_reason),
               "n_output": info.n_output, "n_computed": info.n_computed, "n_preempted": info.n_preempted}
        return out

    @property
    def status(self) -> RequestStatus:
        return self._info()["status"]

    @property
    def finish_reason(self) -> FinishReason:
        return self._info()["finish_reason"]

    @property
    def n_preempted(self) -> int:
        return self._info()["n_preempted"]

    @property
    def done(self) -> bool:
        return self.status in (RequestStatus.FINISHED, RequestStatus.CANCELLED, RequestStatus.OUT_OF_MEMORY)

    @property
    def output(self) -> List[int]:
        if self._final is not None:
            return self._final["output"]
        if self._refused:
            return []
        lib, ctx = capi.load(), self._engine._ctx
        n = ctypes.c_int(0)
        capi.check(lib.imp_request_output(ctx, self.rid, None, 0, ctypes.byref(n)))
        buf = (ctypes.c_int32 * max(n.value, 1))()
        capi.check(lib.imp_request_output(ctx, self.rid, buf, n.value, ctypes.byref(n)))
        return list(buf[:n.value])

    def release(self) -> None:
        """Keep the final state here and let the engine forget the request."""
        if self._final is None and not self._refused:
            info = self._info()
            info["output"] = self.output
            if info["status"] in (RequestStatus.FINISHED, RequestStatus.CANCELLED, RequestStatus.OUT_OF_MEMORY):
                capi.check(capi.load().imp_request_release(self._engine._ctx, self.rid))
                self._final = info


class Model:
    """A model handle: configuration, plan, and where the tensors come from (a folder, or a seed)."""

    def __init__(self, handle):
        self._h = handle

    @classmethod
    def load(cls, model_dir: str) -> "Model":
        h = ctypes.c_void_p()
        capi.model_error(capi.load().imp_model_load(str(model_dir).encode(), ctypes.byref(h)))
        return cls(h)

    @classmethod
    def random(cls, config, seed: int = 0, std: float = 0.02, norm_std: float = 0.01) -> "Model":
        """`config`: a ModelConfig, a config.json dictionary, or a path."""
        if isinstance(config, ModelConfig):
            text = config.to_json()
        elif isinstance(config, dict):
            text = json.dumps(config)
        else:
            text = str(config)
        h = ctypes.c_void_p()
        capi.model_error(capi.load().imp_model_random(text.encode(), int(seed), float(std), float(norm_std), ctypes.byref(h)))
        return cls(h)

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            try:
                capi.load().imp_model_free(h)
            except Exception:
                pass

    @property
    def architecture(self) -> str:
        return capi.text(capi.load().imp_model_arch(self._h))

    @property
    def vocab_size(self) -> int:
        return capi.load().imp_model_vocab_size(self._h)

    @property
    def config(self) -> ModelConfig:
        from ..config.registry import config_class_of
        d = json.loads(capi.text(capi.load().imp_model_config_json(self._h)))
        return config_class_of(d["architectures"][0])(d)

    def plan_json(self) -> Dict[str, Any]:
        return json.loads(capi.text(capi.load().imp_model_plan_json(self._h)))

    def tensor_info(self, compute_dtype: str = "bfloat16") -> Dict[str, Any]:
        c = capi.COMPUTE_FP32 if compute_dtype == "float32" else capi.COMPUTE_BF16
        return json.loads(capi.text(capi.load().imp_model_tensor_info_json(self._h, c)))


class Engine:
    """Model + cache + step function + scheduler + sampler on one GPU (the library's context)."""

    def __init__(self, model: Model, config: Optional[EngineConfig] = None):
        self.config = config or EngineConfig()
        self.model = model
        self._ids: Dict[Hashable, int] = {}     # step_tokens: the caller's request ids -> integers
        self._next_replay_id = 1 << 40
        c = self.config.to_c()
        ctx = ctypes.c_void_p()
        capi.check(capi.load().imp_context_create(model._h, ctypes.byref(c), ctypes.byref(ctx)))
        self._ctx = ctx
        self.vocab_size = model.vocab_size
        self._outs = (capi.ImpStepOutput * max(self.config.max_batch_size * 2, 8))()

    # ------------------------------------------------------------ construction
    @classmethod
    def from_folder(cls, model_dir: str, config: Optional[EngineConfig] = None) -> "Engine":
        return cls(Model.load(model_dir), config)

    @classmethod
    def from_random(cls, model_config, config: Optional[EngineConfig] = None, seed: int = 0, std: float = 0.02,
                    norm_std: float = 0.01) -> "Engine":
        return cls(Model.random(model_config, seed, std, norm_std), config)

    def close(self) -> None:
        ctx, self._ctx = getattr(self, "_ctx", None), None
        if ctx:
            capi.load().imp_context_free(ctx)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def model_config(self) -> ModelConfig:
        return self.model.config

    def info(self) -> Dict[str, Any]:
        """State of the context: cache groups and free pages, run positions, counters."""
        return json.loads(capi.text(capi.load().imp_context_info_json(self._ctx)))

    @property
    def eos_token_ids(self):
        return tuple(self.info()["eos_token_ids"])

    @eos_token_ids.setter
    def eos_token_ids(self, ids) -> None:
        arr, n = capi.int32_array([int(t) for t in ids])
        capi.check(capi.load().imp_context_set_eos(self._ctx, arr, n))

    def free_pages(self) -> int:
        return self.info()["cache"]["free_pages"]

    @property
    def num_pages(self) -> int:
        return self.info()["cache"]["num_pages"]

    def timer_start(self) -> None:
        """Mark the start of a device-timed region on the engine's stream (a CUDA event)."""
        capi.check(capi.load().imp_context_timer_start(self._ctx))

    def timer_stop(self) -> float:
        """Wait for the work queued since `timer_start`; its device time in milliseconds."""
        ms = ctypes.c_float(0.0)
        capi.check(capi.load().imp_context_timer_stop(self._ctx, ctypes.byref(ms)))
        return float(ms.value)

    def check_invariants(self) -> None:
        """The cache manager's invariants (no page lost, held twice or freed twice)."""
        capi.check(capi.load().imp_context_check(self._ctx))

    def reset(self) -> None:
        capi.check(capi.load().imp_context_reset(self._ctx))
        self._ids.clear()

    # ---------------------------------------------------------------- requests
    def submit(self, prompt: Sequence[int], params: Optional[GenerateParams] = None) -> Request:
        """Queue one request; returns its handle (check `.status` for OUT_OF_MEMORY)."""
        p = (params or GenerateParams()).to_c()
        toks, n = capi.int32_array([int(t) for t in prompt])
        rid = ctypes.c_int64(-1)
        rc = capi.load().imp_submit(self._ctx, toks, n, ctypes.byref(p), ctypes.byref(rid))
        if rc == capi.IMP_ERROR_OUT_OF_MEMORY:
            return Request(self, rid.value, prompt, refused=True)
        capi.check(rc)
        return Request(self, rid.value, prompt)

    def cancel(self, request) -> None:
        capi.check(capi.load().imp_cancel(self._ctx, request.rid if isinstance(request, Request) else int(request)))

    def has_work(self) -> bool:
        return bool(capi.load().imp_has_work(self._ctx))

    def _outputs(self, fn) -> List[StepOutput]:
        n = ctypes.c_int(0)
        capi.check(fn(self._ctx, self._outs, len(self._outs), ctypes.byref(n)))
        return [StepOutput(o.id, o.token, bool(o.finished), RequestStatus(o.status), FinishReason(o.finish_reason))
                for o in self._outs[:n.value]]

    def step(self) -> List[StepOutput]:
        """One engine step: schedule, run the batch, sample, finish.  Returns the new tokens."""
        return self._outputs(capi.load().imp_step)

    def drain(self) -> List[StepOutput]:
        """Finish a step that was launched ahead, if any (its requests may all have ended already)."""
        return self._outputs(capi.load().imp_drain)

    def generate(self, prompts: Sequence[Sequence[int]], params=None) -> List[List[int]]:
        """Generate for every prompt (continuous batching inside); returns the new tokens per prompt.
        `params` is one GenerateParams for all prompts or a list with one per prompt."""
        if prompts and isinstance(prompts[0], int):
            raise TypeError("generate takes a list of prompts (each a list of token ids)")
        plist = params if isinstance(params, (list, tuple)) else [params] * len(prompts)
        reqs = [self.submit(p, q) for p, q in zip(prompts, plist)]
        for r in reqs:
            if r.status == RequestStatus.OUT_OF_MEMORY:
                raise MemoryError(f"request {r.rid!r}: prompt plus max_tokens needs more cache pages than the pool holds")
        live = {r.rid for r in reqs}
        while live:
            for o in self.step():
                if o.finished:
                    live.discard(o.rid)
            if live and not self.has_work():
                break
        if not self.has_work():
            self.drain()
        failed = [r.rid for r in reqs if r.status != RequestStatus.FINISHED]
        if failed:
            raise MemoryError(f"{len(failed)} request(s) ran out of cache pages: {failed}")
        outs = [r.output for r in reqs]
        for r in reqs:
            r.release()
        return outs

    # ------------------------------------------------------------- token level
    def _rid(self, rid: Hashable) -> int:
        if rid not in self._ids:
            self._ids[rid] = self._next_replay_id
            self._next_replay_id += 1
        return self._ids[rid]

    def step_tokens(self, entries: Sequence[StepEntry]):
        """Run given tokens as one batch (no scheduling, no sampling).  Returns the logits of the wanted rows
        as a float32 numpy array [wanted, vocab], in the order of the entries and of each `want`."""
        import numpy as np
        n = len(entries)
        arr = (capi.ImpStepEntry * max(n, 1))()
        keep = []
        wanted = 0
        for i, e in enumerate(entries):
            toks, nt = capi.int32_array([int(t) for t in e.tokens])
            want, nw = capi.int32_array([int(w) for w in e.want])
            keep += [toks, want]
            arr[i].id = self._rid(e.rid)
            arr[i].tokens = toks
            arr[i].n_tokens = nt
            arr[i].want = want
            arr[i].n_want = nw
            wanted += nw
        out = np.empty((wanted, self.vocab_size), dtype=np.float32)
        capi.check(capi.load().imp_step_tokens(self._ctx, arr, n, out.ctypes.data_as(ctypes.c_void_p), out.size))
        return out

    def end(self, rid: Hashable) -> None:
        """Give back what a `step_tokens` request holds."""
        capi.check(capi.load().imp_end(self._ctx, self._rid(rid)))
        self._ids.pop(rid, None)
