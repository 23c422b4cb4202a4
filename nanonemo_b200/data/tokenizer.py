"""GPT-2 BPE tokenizer access, loaded lazily.

The reference builds the tiktoken encoder at import time (nanonemo/data/tokenizer.py:12), which
needs the network the first time and makes its loader unimportable offline. Here the encoder is
created on first use only; everything that just needs the constants (the loader, the synthetic
source, shard headers) never touches tiktoken.
"""

from concurrent.futures import ThreadPoolExecutor
from functools import lru_cache

TOKENIZER_NAME = "gpt2"
VOCAB_SIZE = 50257
EOT = 50256


@lru_cache(maxsize=1)
def encoder():
    try:
        import tiktoken

        return tiktoken.get_encoding(TOKENIZER_NAME)
    except Exception as e:  # no package, or no cached vocabulary and no network
        raise RuntimeError(f"GPT-2 tokenizer unavailable ({type(e).__name__}: {e}); "
                           "tokenising text needs tiktoken with a cached gpt2 vocabulary") from e


def encode_doc(text: str) -> list[int]:
    """Token ids of one document followed by end-of-text; special tokens in the text stay plain text."""
    return encoder().encode_ordinary(text) + [EOT]


def encode_batch(texts: list[str], num_threads: int = 8) -> list[list[int]]:
    enc = encoder()
    if hasattr(enc, "encode_ordinary_batch"):
        return [ids + [EOT] for ids in enc.encode_ordinary_batch(texts, num_threads=num_threads)]
    with ThreadPoolExecutor(num_threads) as pool:
        return list(pool.map(encode_doc, texts))


def decode(ids) -> str:
    return encoder().decode(list(ids))
