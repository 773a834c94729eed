"""In-Python use, in the reference's manner (Tokenomos api/llm.py:36-56,71-143,227-234)::

    from tokenomos_b200 import LLM, SamplingParams
    with LLM(path, max_len=4096) as llm:
        outs = llm.generate([[1, 2, 3], "some text"], SamplingParams(max_tokens=32))

``generate`` takes token id lists, or text when the folder has a ``tokenizer.json`` (folders
written by the random-weights mode have none: use id lists). The engine loop runs in a
background thread serving its inbox; an exception there is stored and surfaces in ``wait``.
Stops: the generation config's EOS ids plus any ``stop_token_ids`` given.
"""

from __future__ import annotations

import json
import threading
from concurrent.futures import Future, wait
from dataclasses import dataclass
from pathlib import Path

import torch

from tokenomos_b200 import models
from tokenomos_b200.engine.engine import Engine
from tokenomos_b200.engine.scheduler import Request
from tokenomos_b200.sampling.params import SamplingParams

__all__ = ["LLM", "SamplingParams", "Output"]


@dataclass
class Output:
    text: str
    token_ids: list[int]
    prompt_tokens: int
    finish: str


class LLM:
    def __init__(self, model: str, device: str = "cuda", arch=None, work: str | None = None,
                 **engine_kw):
        """``arch``: a configured declaration (``models.configure(path, work=...)``); ``work``:
        shorthand for the work dtype (``bf16`` or ``fp32``); ``engine_kw`` go to ``Engine``
        (``slots``, ``page``, ``max_len``, ``pages``, ``prefill_budget``, ``graphs``)."""
        self.path = Path(model)
        if arch is None:
            arch = models.configure(model, work=work)
        self.model = models.load(model, device, arch)
        self.tokenizer = None
        tok = self.path / "tokenizer.json"
        if tok.exists():
            from tokenizers import Tokenizer
            self.tokenizer = Tokenizer.from_file(str(tok))
        gen_path = self.path / "generation_config.json"
        gen = json.loads(gen_path.read_text("utf-8")) if gen_path.exists() else {}
        eos = gen.get("eos_token_id", [])
        eos = set(eos if isinstance(eos, list) else [eos])
        self.eos = tuple(sorted(e for e in eos if e is not None))
        self.engine = Engine(self.model, device=device, **engine_kw)
        self._stop, self._error = threading.Event(), None
        self._device = torch.device(device)
        self._thread = threading.Thread(target=self._serve, name="tokenomos-b200-engine", daemon=True)
        self._thread.start()

    def request(self, ids: list[int], p: SamplingParams) -> Request:
        """An engine Request for prompt ``ids`` (stops: the model's EOS plus ``p``'s)."""
        p.validate()
        return Request(
            list(ids), max_new=p.max_tokens, temperature=p.temperature, top_p=p.top_p,
            top_k=p.top_k, min_p=p.min_p, seed=p.seed,
            stop=tuple(dict.fromkeys(self.eos + tuple(p.stop_token_ids))))

    # ---- the serving thread ----

    def _serve(self) -> None:
        try:
            if self._device.index is not None:
                torch.cuda.set_device(self._device)
            self.engine.run(self._stop)
        except BaseException as e:  # noqa: BLE001 - stored for the callers' threads
            self._error = e
            raise

    def submit(self, req: Request) -> Future:
        """Queue one engine request; the future resolves to it once ``req.result`` is set."""
        fut: Future = Future()
        req.on_done = lambda r: fut.set_result(r)
        self.engine.submit(req)
        return fut

    def encode(self, text: str) -> list[int]:
        if self.tokenizer is None:
            raise ValueError(f"{self.path} has no tokenizer.json: pass token id lists")
        return self.tokenizer.encode(text, add_special_tokens=False).ids

    def wait(self, futs: list[Future]) -> list[Request]:
        """Every future's Request; raises if the engine thread died."""
        pending = set(futs)
        while pending:
            if self._error is not None:
                raise RuntimeError("engine thread failed") from self._error
            _, pending = wait(pending, timeout=0.2)
        return [f.result() for f in futs]

    def output(self, req: Request) -> Output:
        r = req.result
        text = ""
        if self.tokenizer is not None:
            text = self.tokenizer.decode(r.tokens, skip_special_tokens=True)
        return Output(text, r.tokens, len(req.prompt), r.finish)

    @property
    def failure(self) -> BaseException | None:
        """What ended the engine thread, or None while it serves."""
        return self._error

    def close(self) -> None:
        self._stop.set()
        self._thread.join()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    # ---- requests ----

    def generate(self, prompts: list, params: SamplingParams | None = None) -> list[Output]:
        """``prompts``: token id lists, or text (tokenized as is)."""
        p = params or SamplingParams()
        futs = [self.submit(self.request(x if isinstance(x, list) else self.encode(x), p))
                for x in prompts]
        return [self.output(r) for r in self.wait(futs)]
