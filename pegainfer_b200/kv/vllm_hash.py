"""Block keys that a vLLM prefill node would register for the same tokens.

When vLLM is the prefill side of a prefill/decode split, its connector stores KV blocks under
vLLM's own prefix-cache hashes.  A decode node finds those blocks by content only if it derives
byte-identical keys.  One vLLM configuration can be reproduced outside vLLM and this module
mirrors exactly that one: ``--prefix-caching-hash-algo xxhash_cbor`` (key = ``xxh3_128`` of the
canonical CBOR encoding, RFC 8949) with ``PYTHONHASHSEED`` set on every vLLM process (the chain
root is ``xxh3_128(cbor(seed_string))``), text-only requests (the third tuple element is null).
Per block the hashed value is the CBOR array ``[parent_hash: bytes, [token, ...], null]``; only
full blocks have a key.

The CBOR subset needed here (unsigned ints, byte strings, text strings, arrays, null) is written
out by hand so that the key derivation has no dependency beyond ``xxhash``.

Reference parity: pegainfer-kv-offload/src/vllm_hash.rs:32-218.
"""
from __future__ import annotations

from typing import Iterable, List, Optional, Sequence

KEY_BYTES = 16
_UINT, _BSTR, _TSTR, _ARRAY = 0, 2, 3, 4
_NULL = b"\xf6"


def cbor_head(major: int, value: int) -> bytes:
    """Canonical (shortest) CBOR head: major type and unsigned argument."""
    m = major << 5
    if value < 24:
        return bytes((m | value,))
    if value <= 0xFF:
        return bytes((m | 0x18, value))
    if value <= 0xFFFF:
        return bytes((m | 0x19,)) + value.to_bytes(2, "big")
    if value <= 0xFFFFFFFF:
        return bytes((m | 0x1A,)) + value.to_bytes(4, "big")
    return bytes((m | 0x1B,)) + value.to_bytes(8, "big")


def _xxh3_128(data: bytes) -> bytes:
    try:
        import xxhash
    except ImportError as exc:  # pragma: no cover - the image ships xxhash
        raise RuntimeError("vLLM-compatible block keys need the `xxhash` package") from exc
    return xxhash.xxh3_128_digest(data)


def encode_block(parent: bytes, token_ids: Sequence[int]) -> bytes:
    out = bytearray(cbor_head(_ARRAY, 3))
    out += cbor_head(_BSTR, len(parent)) + parent
    out += cbor_head(_ARRAY, len(token_ids))
    for t in token_ids:
        out += cbor_head(_UINT, int(t))
    out += _NULL
    return bytes(out)


class VllmBlockHasher:
    """Key chains for one ``(PYTHONHASHSEED, block_size)`` configuration."""

    def __init__(self, python_hash_seed: str, block_size: int):
        if block_size <= 0:
            raise ValueError("block_size must be positive")
        seed = python_hash_seed.encode()
        self.none_hash = _xxh3_128(cbor_head(_TSTR, len(seed)) + seed)
        self.block_size = block_size

    def hash_block(self, parent: Optional[bytes], token_ids: Sequence[int]) -> bytes:
        return _xxh3_128(encode_block(parent if parent is not None else self.none_hash, token_ids))

    def key_chain(self, token_ids: Sequence[int]) -> List[bytes]:
        """One key per FULL block of ``token_ids`` (the partial tail has none)."""
        keys: List[bytes] = []
        parent: Optional[bytes] = None
        bs = self.block_size
        for i in range(len(token_ids) // bs):
            parent = self.hash_block(parent, token_ids[i * bs : (i + 1) * bs])
            keys.append(parent)
        return keys

    def tail_key(self, token_ids: Sequence[int]) -> Optional[bytes]:
        """Key of the partial tail block under the same function (what a P/D tail extension uses)."""
        bs = self.block_size
        full = len(token_ids) // bs
        if len(token_ids) == full * bs:
            return None
        chain = self.key_chain(token_ids)
        return self.hash_block(chain[-1] if chain else None, token_ids[full * bs :])

    def fingerprint(self) -> str:
        """Chain root as hex: prefill and decode side must log the same value at start-up."""
        return self.none_hash.hex()
