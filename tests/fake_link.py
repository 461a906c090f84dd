"""A stand-in for ``tp.PeerLink`` on CPU ranks (gloo): peers' buffers are local staging copies that
travel at every ``exchange``.  Each region of a buffer has one writer (slot s / row block s belongs
to source rank s), so shipping every staged region at every barrier leaves the same contents as
direct peer stores followed by that barrier."""
from __future__ import annotations

import torch
import torch.distributed as dist


class GlooLink:
    def __init__(self, layout: dict, group=None):
        self.group = group
        self.rank, self.size = dist.get_rank(group), dist.get_world_size(group)
        self.layout = layout
        self.mine = {n: self._zeros(shape, dt) for n, (shape, dt) in layout.items()}
        self.staged = {(d, n): self._zeros(shape, dt) for n, (shape, dt) in layout.items()
                       for d in range(self.size) if d != self.rank}
        self.exchanges = 0

    @staticmethod
    def _zeros(shape, dtype):
        if dtype == torch.float8_e4m3fn:
            return torch.zeros(shape, dtype=torch.uint8).view(dtype)
        return torch.zeros(shape, dtype=dtype)

    def buffer(self, r, name):
        return self.mine[name] if r == self.rank else self.staged[(r, name)]

    def local(self, name):
        return self.mine[name]

    def _region(self, name, source):
        """The part of a buffer that rank ``source`` writes in every rank's copy."""
        n0 = self.layout[name][0][0]
        if n0 == self.size:
            return source
        rows = n0 // self.size
        return slice(rows * source, rows * (source + 1))

    def put(self, name, index):
        for d in range(self.size):
            if d != self.rank:
                self.staged[(d, name)][index].copy_(self.mine[name][index])

    @staticmethod
    def _bytes(t):
        return t.view(torch.uint8) if t.dtype == torch.float8_e4m3fn else t

    def exchange(self, maxima=None):
        self.exchanges += 1
        for name in self.layout:
            work, landing = [], []
            for d in range(self.size):
                if d == self.rank:
                    continue
                out = self._bytes(self.staged[(d, name)][self._region(name, self.rank)]).contiguous()
                work.append(dist.isend(out, dist.get_global_rank(self.group, d) if self.group else d, group=self.group))
                buf = torch.empty_like(self._bytes(self.mine[name][self._region(name, d)]).contiguous())
                work.append(dist.irecv(buf, dist.get_global_rank(self.group, d) if self.group else d, group=self.group))
                landing.append((d, buf))
            for w in work:
                w.wait()
            for d, buf in landing:
                self._bytes(self.mine[name])[self._region(name, d)].copy_(buf)
        if maxima is not None:
            name, out = maxima
            out.copy_(self.mine[name].amax(0))

    def check(self):
        return None
