"""A collective program as an object that can be registered and called (the reference's ``pccl/lang/operator.py``
is an empty file; its engine exposes ``regOp(name, json)`` / ``exeOp(name, in, out)``, csrc/python_api.cc:13-20).

    op = Operator.from_algorithm("ring_allreduce", world, channels=2)     # or Operator("mine", my_ir)
    op.register(engine)
    op(x)                       # in place;  op(x, out, width=8, lane=1) for the runtime resource controls
"""
from __future__ import annotations

import json
from typing import Optional

from .algorithms import build
from .ir import CollectiveIR
from .lower import to_schedule
from .verify import verify


class Operator:
    def __init__(self, name: str, ir: CollectiveIR, check: bool = True):
        if check:
            verify(ir).raise_if_failed()
        self.name, self.ir = name, ir
        self._schedule: Optional[dict] = None
        self._engine = None

    @classmethod
    def from_algorithm(cls, algorithm: str, world: int, name: Optional[str] = None, **kw) -> "Operator":
        return cls(name or algorithm, build(algorithm, world, **kw))

    @classmethod
    def synthesized(cls, collective: str, topology, nbytes: int, name: Optional[str] = None, **kw) -> "Operator":
        """A MILP-synthesised schedule for ``collective`` on ``topology`` (see ``pccl_b200.synth.synthesize``)."""
        from ..synth import synthesize
        res = synthesize(collective, topology, nbytes, **kw)
        return cls(name or res.ir.name, res.ir, check=False)     # the synthesiser verified it

    @classmethod
    def best(cls, collective: str, topology, nbytes: int, name: Optional[str] = None, **kw) -> "Operator":
        """The cheapest program for ``collective`` on ``topology`` at this size under the cost model
        (``pccl_b200.synth.choose``; ``include_milp=True`` also prices a synthesised schedule)."""
        from ..synth import choose
        ranked = choose(collective, topology, nbytes, **kw)
        if not ranked:
            raise ValueError(f"no library algorithm for {collective} fits this topology (try include_milp=True)")
        chosen, est, ir = ranked[0]
        op = cls(name or chosen, ir, check=False)
        op.estimate = est
        return op

    @property
    def collective(self) -> str:
        return self.ir.collective

    def schedule(self) -> dict:
        """The lowered JSON schedule (cached)."""
        if self._schedule is None:
            self._schedule = to_schedule(self.ir)
        return self._schedule

    def save(self, path: str) -> str:
        with open(path, "w") as f:
            json.dump(self.schedule(), f)
        return path

    def register(self, engine) -> "Operator":
        engine.regOp(self.name, self.schedule())
        self._engine = engine
        return self

    def __call__(self, input, output=None, **kw) -> int:
        if self._engine is None:
            raise RuntimeError(f"operator '{self.name}' is not registered with an engine")
        return self._engine.exeOp(self.name, input, output, **kw)


__all__ = ["Operator"]
