"""Helpers shared by the tests: paired GPU/oracle views over the same storage contents."""
from __future__ import annotations

import numpy as np

from oracle import oracle as O


class Pair:
    """A strided view held twice: as a ClTensor over an uploaded storage and as an oracle
    View over a private numpy copy of that storage. After the same operation on both,
    `check()` compares the WHOLE storages, so a stray write outside the view is caught."""

    def __init__(self, base: np.ndarray, offset: int = 0, sizes=None, strides=None):
        import cltorch_b200 as cl
        self.host = np.ascontiguousarray(base, dtype=np.float32).reshape(-1).copy()
        sizes = list(base.shape if sizes is None else sizes)
        self.view = O.View(self.host, offset, sizes, strides)
        self.storage = cl.ClStorage(self.host)
        self.cl = cl.ClTensor(self.storage, offset + 1, sizes, self.view.strides)

    def device_storage(self) -> np.ndarray:
        return self.storage.float()

    def check(self, max_ulp: int = 0, what: str = ""):
        got = self.device_storage()
        d = O.ulp_diff(got, self.host)
        worst = int(d.max()) if d.size else 0
        assert worst <= max_ulp, f"{what}: max ulp distance {worst} > {max_ulp} at flat index {int(d.argmax())}: " \
                                 f"gpu={got.reshape(-1)[int(d.argmax())]!r} oracle={self.host[int(d.argmax())]!r}"


def rng_uniform(seed: int, shape, lo=0.0, hi=1.0) -> np.ndarray:
    g = np.random.Generator(np.random.PCG64(seed))
    return (g.random(shape, dtype=np.float32) * np.float32(hi - lo) + np.float32(lo)).astype(np.float32)
