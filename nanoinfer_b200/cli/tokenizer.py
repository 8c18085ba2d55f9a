"""Text <-> token ids for the command line. Uses ``tokenizer.json`` of the model folder (through the
``tokenizers`` package) when both exist; otherwise prompts are given as token ids."""
from __future__ import annotations

import os
import sys
from typing import List, Optional


class IdTokenizer:
    """No vocabulary: a prompt is a list of ids ("5 17 3" or "5,17,3"); output is printed as ids."""
    eos_token_id = None

    def encode(self, text: str) -> List[int]:
        try:
            return [int(t) for t in text.replace(",", " ").split()]
        except ValueError:
            raise ValueError(f"the model folder has no usable tokenizer.json, so a prompt is a list of token ids "
                             f"(\"5 17 3\"); got {text!r}") from None

    def decode(self, ids) -> str:
        return " ".join(str(int(i)) for i in ids)


class JsonTokenizer:
    def __init__(self, path: str, eos_token_id: Optional[int]):
        from tokenizers import Tokenizer
        self._tok = Tokenizer.from_file(path)
        self.eos_token_id = eos_token_id

    def encode(self, text: str) -> List[int]:
        return self._tok.encode(text).ids

    def decode(self, ids) -> str:
        return self._tok.decode([int(i) for i in ids], skip_special_tokens=True)


def load_tokenizer(model_dir: str, eos_token_id: int = -1):
    path = os.path.join(model_dir, "tokenizer.json")
    if os.path.isfile(path):
        try:
            return JsonTokenizer(path, eos_token_id if eos_token_id >= 0 else None)
        except ImportError:
            print(f"{path} is there but the 'tokenizers' package is not: prompts are read as token ids",
                  file=sys.stderr)
    return IdTokenizer()
