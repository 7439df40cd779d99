"""The Python entry point, in the manner of the reference's
``IntQwen3(artifact_dir, backend)`` with ``.forward``, ``.generate(ids, max_new,
guard, chunk_valid, stop_at_eos, use_graph)`` and ``.greedy_pick``
(src/detllm/model.py:105-106, 220-222, 482-495; usage in README.md:272-281).

``load(model_dir, dtype)`` reads config.json, picks the model through the
registry, loads the weights by name and returns an ``LM``.  ``LM.generate``
keeps the reference's argument names and return shape (tokens ``[B, max_new]``
and the list of per-step logits) and adds what the reference lacks: stop
tokens that are honoured, temperature and seed.
"""

from __future__ import annotations

from typing import List, Optional, Sequence, Union

import torch

from .engine.assembly import CausalLM, declare_weights
from .engine.engine import Engine
from .engine.generate import GenerationResult, generate as run_generation
from .kernels import Kernels
from .parts.base import Runtime
from .registry import read_config
from .weights import load_weights, random_weights

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32,
           "fp32": torch.float32, torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


def canonical_dtype(dtype) -> torch.dtype:
    """Normalise a dtype name or raise (as the reference's ``canonical_backend`` does for
    backend names, src/detllm/backends.py:27-34)."""
    try:
        return _DTYPES[dtype]
    except KeyError:
        raise ValueError(f"unknown dtype {dtype!r}; use 'bfloat16' or 'float32'") from None


def build_model(config, weights, dtype, device="cuda:0", arch=None) -> CausalLM:
    dtype = canonical_dtype(dtype)
    device = torch.device(device)
    rt = Runtime(device=device, dtype=dtype, kernels=Kernels(dtype, device))
    spec = config.to_model_spec()
    if arch is not None and arch.build_model is not None:
        return arch.build_model(spec, weights, rt)
    return CausalLM(spec, weights, rt)


class LM:
    """A loaded model with its engine (cache, step function, decode graphs)."""

    def __init__(self, model: CausalLM, config, max_tokens: int = 8192, max_seqs: Optional[int] = None,
                 max_seq_len: Optional[int] = None, use_graph: bool = True):
        self.model = model
        self.config = config
        self.spec = model.spec
        self.device = model.rt.device
        self.engine = Engine(model, max_tokens, max_seqs=max_seqs, max_seq_len=max_seq_len, use_graph=use_graph)

    # the reference's names -------------------------------------------------------
    def greedy_pick(self, logits_row: torch.Tensor) -> torch.Tensor:
        """Argmax with lowest-token-id tie-break over ``[B, vocab]`` logits (src/detllm/model.py:482-490)."""
        return self.model.rt.kernels.sample(logits_row.contiguous().float(), 0.0, None).to(torch.int64)

    @torch.no_grad()
    def generate(self, ids: Union[torch.Tensor, Sequence[Sequence[int]]], max_new: int,
                 chunk_valid: Optional[torch.Tensor] = None, stop_at_eos: bool = False,
                 use_graph: bool = True, temperature: float = 0.0, seed: int = 0,
                 stop_token_ids: Optional[Sequence[int]] = None, return_logits: bool = True,
                 batch_size: Optional[int] = None):
        """Generate ``max_new`` tokens per prompt.

        ``ids``: int64 ``[B, T0]`` right-padded with ``chunk_valid`` marking real tokens (the
        reference's form), or a list of token lists.  Returns ``(tokens [B, max_new] int64,
        step_logits)``: positions after a sequence's end hold -1; ``step_logits[i]`` is
        ``[B, vocab]`` float32 for the i-th generated token (rows of ended sequences are zero)."""
        prompts = self._prompts(ids, chunk_valid)
        stops = list(stop_token_ids) if stop_token_ids is not None else (
            list(self.spec.stop_token_ids) if stop_at_eos else [])
        self.engine.use_graph = use_graph and self.device.type == "cuda"
        res = run_generation(self.engine, prompts, max_new, temperature=temperature, seed=seed,
                             stop_token_ids=stops, return_logits=return_logits, batch_size=batch_size)
        B = len(prompts)
        toks = torch.full((B, max_new), -1, dtype=torch.int64)
        for r in res:
            toks[r.request, :len(r.tokens)] = torch.tensor(r.tokens, dtype=torch.int64)
        step_logits = []
        if return_logits:
            V = self.spec.vocab_size
            for i in range(max_new):
                rows = [r.logits[i] if i < len(r.logits) else torch.zeros(V, device=self.device) for r in res]
                step_logits.append(torch.stack(rows))
        return toks, step_logits

    def generate_requests(self, prompts: Sequence[Sequence[int]], max_new: int, **kw) -> List[GenerationResult]:
        """The same loop, returning one ``GenerationResult`` per request."""
        return run_generation(self.engine, [list(p) for p in prompts], max_new, **kw)

    @staticmethod
    def _prompts(ids, chunk_valid) -> List[List[int]]:
        if isinstance(ids, torch.Tensor):
            ids = ids.detach().cpu()
            if ids.dim() == 1:
                ids = ids[None]
            if chunk_valid is None:
                return [row.tolist() for row in ids]
            cv = chunk_valid.detach().cpu().bool()
            return [row[m].tolist() for row, m in zip(ids, cv)]
        return [list(map(int, p)) for p in ids]


def load(model_dir: str, dtype="bfloat16", device="cuda:0", max_tokens: int = 8192,
         max_seqs: Optional[int] = None, max_seq_len: Optional[int] = None, use_graph: bool = True) -> LM:
    """Load the model folder ``model_dir`` (config.json, model.safetensors)."""
    arch, config = read_config(model_dir)
    spec = config.to_model_spec()
    weights = load_weights(model_dir, declare_weights(spec), torch.device(device))
    model = build_model(config, weights, dtype, device, arch)
    del weights
    return LM(model, config, max_tokens=max_tokens, max_seqs=max_seqs, max_seq_len=max_seq_len,
              use_graph=use_graph)


def from_random(config, seed: int = 0, dtype="bfloat16", device="cuda:0", std: Optional[float] = None,
                **engine_kw) -> LM:
    """A model of ``config``'s sizes with seeded random weights drawn on the device (no folder is
    written; for sizes whose files would be too large to make first)."""
    dt = canonical_dtype(dtype)
    spec = config.to_model_spec()
    weights = random_weights(declare_weights(spec), seed, spec.init_std if std is None else std,
                             dtype=dt, device=device)
    model = build_model(config, weights, dt, device)
    del weights
    return LM(model, config, **engine_kw)
