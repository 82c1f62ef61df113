"""Host transcript mirror (verinf_b200/transcript.py) against the reference's coins
(layergkr/transcript.py:96-112; golden `coins_seed0_sc24` drawn by the reference's class)."""
import blake3

from verinf_b200.transcript import P, Transcript, seeded_coins


def test_seeded_coins_equal_reference_golden(golden):
    want = [int(v) for v in golden.hash_vectors["coins_seed0_sc24"]]
    assert seeded_coins(b"bench/sumcheck", 0, "sc", 24) == want


def test_coin_formula_and_state_chaining():
    t = Transcript(b"dom")
    t.absorb("a", b"xyz")
    h = blake3.blake3(b"dom")
    h.update((1).to_bytes(2, "little") + b"a" + (3).to_bytes(8, "little") + b"xyz")
    state = h.digest()
    c = t.coin("lab", 2)
    assert c == [int.from_bytes(blake3.blake3(state + b"lab" + i.to_bytes(8, "little")).digest()[:16], "little") % P
                 for i in range(2)]
    # a coin call advances the state: the next draw differs, and is back-date proof
    h.update(b"\x00coin" + (3).to_bytes(2, "little") + b"lab")
    assert t.digest() == h.digest()
    assert t.coin("lab", 1) != c[:1]
    assert [e[0] for e in t.log] == ["absorb", "coin", "coin"]
