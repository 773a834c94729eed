"""The Python entry point: ``LLM(path).generate(prompts, SamplingParams(...))``.

    from tokenomos_b200 import LLM, SamplingParams
    with LLM(folder, max_len=4096) as llm:
        replies = llm.generate([[1, 2, 3], [7, 8]], SamplingParams(max_tokens=32, temperature=0.8))

The names (``LLM``, ``SamplingParams``, ``Output``, ``generate``, ``submit``, ``wait``,
``stream``) and the meaning of the options are the reference's (Tokenomos api/llm.py:36-56,
71-143, 227-265); what is behind them is this engine. An ``LLM`` owns the loaded model, an
``Engine`` and one worker thread that runs the engine's loop. Callers hand requests over through
the engine's inbox and get them back through futures, so any number of threads may call
``generate`` at once and their requests share the running batch.

Prompts are lists of token ids. Text is accepted when the folder has a ``tokenizer.json``
(folders written by the random-weights mode have none). A reply ends at ``max_tokens``, at one
of the folder's end-of-sequence ids (``generation_config.json``), or at one of
``SamplingParams.stop_token_ids``; the stop token is part of the reply.
"""

from __future__ import annotations

import json
import queue
import threading
from concurrent.futures import Future
from concurrent.futures import TimeoutError as FutureTimeout
from dataclasses import dataclass
from pathlib import Path

import torch

from tokenomos_b200 import models
from tokenomos_b200.engine.engine import Engine
from tokenomos_b200.engine.scheduler import Request
from tokenomos_b200.sampling.params import SamplingParams

__all__ = ["LLM", "SamplingParams", "Output"]

# how often a caller that waits looks whether the worker is still alive
POLL_S = 0.1


@dataclass
class Output:
    text: str
    token_ids: list[int]
    prompt_tokens: int
    finish: str


def folder_stop_ids(folder: Path) -> tuple[int, ...]:
    """The end-of-sequence ids ``generation_config.json`` names: one id, a list, or none."""
    path = folder / "generation_config.json"
    if not path.is_file():
        return ()
    named = json.loads(path.read_text("utf-8")).get("eos_token_id")
    if named is None:
        return ()
    ids = named if isinstance(named, (list, tuple)) else (named,)
    return tuple(sorted({int(i) for i in ids if i is not None}))


class _Worker(threading.Thread):
    """The thread the engine's loop lives on. Whatever ends the loop other than ``halt`` is
    kept in ``error`` for the callers, who would otherwise wait for futures nobody resolves."""

    def __init__(self, engine: Engine, device: torch.device):
        super().__init__(name="tokenomos-b200-engine", daemon=True)
        self.engine, self.device = engine, device
        self.halted = threading.Event()
        self.error: BaseException | None = None

    def run(self) -> None:
        try:
            if self.device.type == "cuda" and self.device.index is not None:
                torch.cuda.set_device(self.device)
            self.engine.run(self.halted)
        except BaseException as exc:  # noqa: BLE001 - handed to the waiting callers
            self.error = exc

    def halt(self) -> None:
        self.halted.set()
        self.join()


class LLM:
    def __init__(self, model: str, device: str = "cuda", arch=None, work: str | None = None,
                 **engine_kw):
        """``model``: a folder with config.json and safetensors. ``arch``: what
        ``models.configure(folder, work=...)`` returned, when the caller configured it; ``work``
        alone picks the work dtype (``bf16``, the default, or ``fp32``). Every other keyword goes
        to ``Engine``: ``slots``, ``page``, ``max_len``, ``pages``, ``prefill_budget``,
        ``graphs``, ``warmup``."""
        self.path = Path(model)
        self._device = torch.device(device)
        self.model = models.load(model, device, arch or models.configure(model, work=work))
        self.tokenizer = self._tokenizer()
        self.eos = folder_stop_ids(self.path)
        self.engine = Engine(self.model, device=device, **engine_kw)
        self._worker = _Worker(self.engine, self._device)
        self._worker.start()

    def _tokenizer(self):
        path = self.path / "tokenizer.json"
        if not path.is_file():
            return None
        from tokenizers import Tokenizer
        return Tokenizer.from_file(str(path))

    # ---- one request ----

    def encode(self, text: str) -> list[int]:
        if self.tokenizer is None:
            raise ValueError(f"{self.path} has no tokenizer.json: pass token id lists")
        return self.tokenizer.encode(text, add_special_tokens=False).ids

    def request(self, ids: list[int], p: SamplingParams) -> Request:
        """The engine request for one prompt: ``p``'s options, and as stops the folder's
        end-of-sequence ids followed by ``p.stop_token_ids`` (each id once)."""
        p.validate()
        stops = list(self.eos)
        stops.extend(t for t in p.stop_token_ids if t not in stops)
        return Request(prompt=list(ids), max_new=p.max_tokens, temperature=p.temperature,
                       top_p=p.top_p, top_k=p.top_k, min_p=p.min_p, seed=p.seed, stop=tuple(stops))

    def submit(self, req: Request) -> Future:
        """Hand ``req`` to the engine. The future's result is ``req`` itself, with ``result``
        filled in, as soon as the engine has finished it. A request the engine can never serve
        raises here, in the caller's thread."""
        self._check_worker()
        done: Future = Future()
        req.on_done = done.set_result
        self.engine.submit(req)
        return done

    def wait(self, futs: list[Future]) -> list[Request]:
        """The finished requests behind ``futs``, in their order. Raises ``RuntimeError`` (with
        the cause chained) if the engine's thread has died, instead of waiting for ever."""
        finished = []
        for fut in futs:
            while True:
                try:
                    finished.append(fut.result(timeout=POLL_S))
                    break
                except FutureTimeout:
                    self._check_worker()
        return finished

    def output(self, req: Request) -> Output:
        reply = req.result
        text = self.tokenizer.decode(reply.tokens, skip_special_tokens=True) if self.tokenizer else ""
        return Output(text=text, token_ids=reply.tokens, prompt_tokens=len(req.prompt),
                      finish=reply.finish)

    # ---- many ----

    def generate(self, prompts: list, params: SamplingParams | None = None) -> list[Output]:
        """One reply per prompt, in order. A prompt is a list of token ids, or text."""
        params = params or SamplingParams()
        futs = [self.submit(self.request(self._ids(prompt), params)) for prompt in prompts]
        return [self.output(req) for req in self.wait(futs)]

    def stream(self, prompt, params: SamplingParams | None = None):
        """Yields the reply's token ids in runs, as the engine delivers them (the host reads a
        step's tokens while the next step runs). The runs joined are ``generate``'s reply."""
        runs: queue.Queue = queue.Queue()
        req = self.request(self._ids(prompt), params or SamplingParams())
        req.on_tokens = lambda toks: runs.put(list(toks))
        fut = self.submit(req)
        while True:
            try:
                yield runs.get(timeout=POLL_S)
            except queue.Empty:
                self._check_worker()
                if fut.done() and runs.empty():
                    return

    def _ids(self, prompt) -> list[int]:
        return self.encode(prompt) if isinstance(prompt, str) else list(prompt)

    # ---- the worker ----

    @property
    def failure(self) -> BaseException | None:
        """The exception that ended the engine's thread; None while it serves."""
        return self._worker.error

    def _check_worker(self) -> None:
        if self._worker.error is not None:
            raise RuntimeError("engine thread failed") from self._worker.error

    def close(self) -> None:
        self._worker.halt()

    def __enter__(self) -> "LLM":
        return self

    def __exit__(self, *exc) -> None:
        self.close()
