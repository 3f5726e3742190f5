"""Speculative-decoding configuration objects (python/yirage/speculative.py).  The
configs exist so that callers can construct them; the speculative task kernels
themselves are outside the decode hot path and are not built."""
from dataclasses import dataclass
from typing import Literal


@dataclass
class SpecDecodeConfig:
    method: str


@dataclass
class LookaheadConfig(SpecDecodeConfig):
    method: Literal["lookahead"] = "lookahead"
    spec_length: int = 7


@dataclass
class PromptLookupConfig(SpecDecodeConfig):
    method: Literal["promptlookup"] = "promptlookup"
    ngram_size: int = 3
    spec_length: int = 5


def spec_decode_class(spec_decode: str, ngram_size: int, spec_length: int):
    if spec_decode == "lookahead":
        return LookaheadConfig(spec_length=spec_length)
    elif spec_decode == "promptlookup":
        return PromptLookupConfig(ngram_size=ngram_size, spec_length=spec_length)
    elif spec_decode is None:
        return None
    raise NotImplementedError(f"Spec decode method {spec_decode} not implemented")
