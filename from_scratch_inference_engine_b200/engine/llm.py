"""`LLM`: a model folder in, generated token ids (or text) out.

Names and defaults as the reference wrapper (python/engine/llm.py:33-76): `LLM(model_dir,
block_size=16, num_blocks=2048, seed=0, max_batch=256, eos_id=None, enable_prefix_cache=
True)`, `GenerationConfig(max_tokens=64, temperature=0.0, top_k=0, top_p=1.0)`,
`generate_ids`, `generate`.  `quantize` is not taken: quantised weights are outside this
engine.  Added: `dtype`, `device`, `max_step_tokens`.
"""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import List, Optional, Sequence

from ..sampling.sampler import SamplingParams
from .engine import Engine, LoadedModel


def read_eos_id(model_dir) -> int:
    """End-of-sequence id from generation_config.json, then config.json; the first element
    of a list; -1 if neither names one (python/engine/llm.py:18-30)."""
    for name in ("generation_config.json", "config.json"):
        path = Path(model_dir) / name
        if not path.exists():
            continue
        eos = json.loads(path.read_text(encoding="utf-8")).get("eos_token_id")
        if isinstance(eos, list):
            eos = eos[0] if eos else None
        if eos is not None:
            return int(eos)
    return -1


@dataclass
class GenerationConfig:
    max_tokens: int = 64
    temperature: float = 0.0     # <= 0 is greedy
    top_k: int = 0
    top_p: float = 1.0
    seed: Optional[int] = None


class LLM:
    def __init__(self, model_dir, *, block_size: int = 16, num_blocks: int = 2048, seed: int = 0,
                 max_batch: int = 256, eos_id: Optional[int] = None,
                 enable_prefix_cache: bool = True, dtype="bfloat16", device="cuda:0",
                 max_step_tokens: int = 2048):
        self.model_dir = Path(model_dir)
        self.model = LoadedModel.from_pretrained(model_dir, dtype=dtype, device=device,
                                                 max_positions=block_size * num_blocks)
        self.engine = Engine(self.model, block_size, num_blocks, seed, max_batch,
                             enable_prefix_cache, max_step_tokens)
        self.eos_id = read_eos_id(model_dir) if eos_id is None else eos_id
        self._tokenizer = None

    @staticmethod
    def _params(config: GenerationConfig) -> SamplingParams:
        return SamplingParams(config.temperature, config.top_k, config.top_p, config.seed)

    def generate_ids(self, prompt_ids: Sequence[int],
                     config: Optional[GenerationConfig] = None) -> List[int]:
        config = config or GenerationConfig()
        return self.engine.generate(list(prompt_ids), self._params(config), config.max_tokens,
                                    self.eos_id)

    def generate_batch(self, prompts: Sequence[Sequence[int]],
                       config: Optional[GenerationConfig] = None) -> List[List[int]]:
        """Submit all prompts up front and run them together (the reference's benchmark
        drives its engine this way, benchmarks/harness/bench_engine.py:48-75)."""
        config = config or GenerationConfig()
        ids = [self.engine.add_request(list(p), self._params(config), config.max_tokens,
                                       self.eos_id) for p in prompts]
        self.engine.run_until_done()
        return [list(self.engine.output(i)) for i in ids]

    @property
    def tokenizer(self):
        if self._tokenizer is None:
            path = self.model_dir / "tokenizer.json"
            if not path.exists():
                raise FileNotFoundError(f"{path} is missing: text prompts need the model's "
                                        f"tokenizer; use generate_ids with token ids")
            from tokenizers import Tokenizer      # the reference's choice (tokenizer.py:14-32)
            self._tokenizer = Tokenizer.from_file(str(path))
        return self._tokenizer

    def generate(self, prompt: str, config: Optional[GenerationConfig] = None) -> str:
        ids = self.tokenizer.encode(prompt).ids
        return self.tokenizer.decode(self.generate_ids(ids, config))
