"""std::mt19937_64 and the uniform draw the reference makes from it: the top
53 bits of one output, scaled (crates/nncpu/src/session/sample.rs:8-55)."""
from __future__ import annotations

_M = (1 << 64) - 1
_NN, _MM = 312, 156


class Mt19937_64:
    def __init__(self, seed: int):
        mt = [seed & _M]
        for i in range(1, _NN):
            prev = mt[i - 1]
            mt.append((6364136223846793005 * (prev ^ (prev >> 62)) + i) & _M)
        self._mt = mt
        self._idx = _NN

    def _refill(self) -> None:
        mt = self._mt
        for i in range(_NN):
            x = (mt[i] & 0xFFFFFFFF80000000) | (mt[(i + 1) % _NN] & 0x7FFFFFFF)
            mt[i] = mt[(i + _MM) % _NN] ^ (x >> 1) ^ (0xB5026F5AA96619E9 if x & 1 else 0)
        self._idx = 0

    def next_u64(self) -> int:
        if self._idx >= _NN:
            self._refill()
        x = self._mt[self._idx]
        self._idx += 1
        x ^= (x >> 29) & 0x5555555555555555
        x ^= (x << 17) & 0x71D67FFFEDA60000
        x ^= (x << 37) & 0xFFF7EEE000000000
        x ^= x >> 43
        return x & _M

    def uniform(self, b: float = 1.0) -> float:
        """Uniform in [0, b)."""
        return float(self.next_u64() >> 11) * (1.0 / 9007199254740992.0) * b
