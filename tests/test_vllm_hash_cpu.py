"""vLLM-compatible block keys: the hand-written canonical CBOR must equal what a CBOR library
produces for the same Python values (that is what vLLM hashes), and the chain must behave like
vLLM's: parent-linked, full blocks only, seed-dependent root."""
import pytest

from pegainfer_b200.kv.vllm_hash import VllmBlockHasher, cbor_head, encode_block

cbor2 = pytest.importorskip("cbor2")
xxhash = pytest.importorskip("xxhash")


def test_cbor_heads_are_canonical():
    for v in (0, 1, 23, 24, 255, 256, 65535, 65536, 2**32 - 1, 2**32, 151935):
        assert cbor_head(0, v) == cbor2.dumps(v, canonical=True)
    assert cbor_head(3, 2) + b"42" == cbor2.dumps("42", canonical=True)


def test_block_encoding_matches_a_cbor_library():
    parent = bytes(range(16))
    toks = [0, 5, 23, 24, 300, 70000, 151935, 2**31]
    assert encode_block(parent, toks) == cbor2.dumps((parent, tuple(toks), None), canonical=True)


def test_key_chain_follows_vllm_rules():
    h = VllmBlockHasher("0", 4)
    assert h.none_hash == xxhash.xxh3_128_digest(cbor2.dumps("0", canonical=True))
    toks = list(range(100, 111))  # two full blocks and a tail of three
    chain = h.key_chain(toks)
    assert len(chain) == 2 and all(len(k) == 16 for k in chain)
    assert chain[0] == xxhash.xxh3_128_digest(cbor2.dumps((h.none_hash, tuple(toks[:4]), None), canonical=True))
    assert chain[1] == xxhash.xxh3_128_digest(cbor2.dumps((chain[0], tuple(toks[4:8]), None), canonical=True))
    # prefix property: a longer sequence keeps the keys of its prefix; a changed token changes every later key
    assert h.key_chain(toks + [1, 2, 3, 4, 5])[:2] == chain
    other = list(toks)
    other[1] += 1
    assert h.key_chain(other)[0] != chain[0] and h.key_chain(other)[1] != chain[1]
    assert h.tail_key(toks) == h.hash_block(chain[1], toks[8:]) and h.tail_key(toks[:8]) is None
    # another seed is another key space
    assert VllmBlockHasher("1", 4).key_chain(toks)[0] != chain[0]
    assert VllmBlockHasher("0", 4).fingerprint() == h.fingerprint()
