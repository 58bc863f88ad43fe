"""Tokenizers of the reference (src/tokenizer.jl).  Token ids are 0-based here; tokens are `bytes`
(the reference's Strings may hold arbitrary bytes, e.g. the <0xNN> byte tokens)."""
from dataclasses import dataclass
from typing import Dict, List


class Tokenizer:
    pass


@dataclass
class BPETokenizer(Tokenizer):
    """src/tokenizer.jl:3-9."""
    id_to_token: List[bytes]
    token_to_id: Dict[bytes, int]
    token_scores: List[float]
    bos_token_id: int
    eos_token_id: int


@dataclass
class CharTokenizer(Tokenizer):
    """src/tokenizer.jl:59-64."""
    id_to_token: List[str]
    token_to_id: Dict[str, int]
    bos_token_id: int
    eos_token_id: int

    @staticmethod
    def from_text(text: str) -> "CharTokenizer":
        """CharTokenizer(text) (src/tokenizer.jl:66-80): sorted distinct characters, then <s> and </s>."""
        id_to_token = sorted(set(text)) + ["<s>", "</s>"]
        token_to_id = {t: i for i, t in enumerate(id_to_token)}
        return CharTokenizer(id_to_token, token_to_id, len(id_to_token) - 2, len(id_to_token) - 1)


def encode(text, tokenizer, pad_input: bool = True) -> List[int]:
    """encode(text, tokenizer) (src/tokenizer.jl:11-57 for BPE, :82-84 for characters)."""
    if isinstance(tokenizer, CharTokenizer):
        return [tokenizer.token_to_id[ch] for ch in text]
    data = text.encode("utf-8") if isinstance(text, str) else bytes(text)
    tokens: List[int] = []
    if len(data) == 0:
        return tokens
    t2i, i2t, scores = tokenizer.token_to_id, tokenizer.id_to_token, tokenizer.token_scores
    if pad_input:
        tokens.append(t2i[b" "])
    for b in data:  # every code unit on its own
        tokens.append(t2i[bytes([b])])
    while True:  # merge the best-scoring adjacent pair until none is in the vocabulary
        best_score, best_id, best_idx = float("-inf"), -1, -1
        for i in range(len(tokens) - 1):
            tid = t2i.get(i2t[tokens[i]] + i2t[tokens[i + 1]])
            if tid is not None and scores[tid] > best_score:
                best_score, best_id, best_idx = scores[tid], tid, i
        if best_idx == -1:
            break
        tokens[best_idx] = best_id
        del tokens[best_idx + 1]
    return tokens
