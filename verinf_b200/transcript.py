"""Host-side Fiat-Shamir transcript with the reference's interface and bytes
(layergkr/transcript.py:70-124): BLAKE3 over an append-only log, challenges
`coin i = int(blake3(state || label || i_le8)[:16], little) mod p`.

The reference's prover keeps using its own class; this mirror exists so that the benchmark and
the sharded sumcheck can draw the seeded challenges of a workload (e.g.
`Transcript(b"bench/sumcheck")`, absorb("seed", seed_le8), coin("sc", 24)) without the reference
tree on the path.  Hashing uses the `blake3` package, as the reference does.
"""
from typing import List, Sequence

import blake3

P = (1 << 64) - (1 << 32) + 1


class Transcript:
    def __init__(self, domain: bytes = b"layergkr/v0"):
        self._h = blake3.blake3(domain)
        self.log: List[tuple] = []

    def absorb(self, label: str, data: bytes) -> None:
        self._h.update(len(label).to_bytes(2, "little") + label.encode())
        self._h.update(len(data).to_bytes(8, "little") + data)
        self.log.append(("absorb", label, data))

    def absorb_root(self, label: str, root: bytes) -> None:
        self.absorb(label, root)

    def absorb_ints(self, label: str, values: Sequence[int]) -> None:
        self.absorb(label, b"".join(int(v).to_bytes(8, "little") for v in values))

    def coin(self, label: str, count: int = 1) -> List[int]:
        state = self._h.digest()
        self._h.update(b"\x00coin" + len(label).to_bytes(2, "little") + label.encode())
        self.log.append(("coin", label, count))
        return [int.from_bytes(blake3.blake3(state + label.encode() + i.to_bytes(8, "little")).digest()[:16],
                               "little") % P for i in range(count)]

    def coin_bytes(self, label: str) -> bytes:
        state = self._h.digest()
        self._h.update(b"\x00coin" + len(label).to_bytes(2, "little") + label.encode())
        self.log.append(("coin", label, 0))
        return blake3.blake3(state + label.encode() + b"cols").digest()

    def digest(self) -> bytes:
        return self._h.digest()


def seeded_coins(domain: bytes, seed: int, label: str, count: int) -> List[int]:
    """The challenge schedule of the seeded workloads: absorb the 8-byte seed, draw `count` coins."""
    t = Transcript(domain)
    t.absorb("seed", int(seed).to_bytes(8, "little"))
    return t.coin(label, count)
