"""Plain-Python configuration base shared by the four model families.

The reference keeps four independent classes with hand-written ``__repr__`` methods
(optimus/models/*/configuration_*.py); here one base provides the printing, dict round trip
and the pipeline/expert divisibility checks.
"""
from __future__ import annotations

import copy


class ParallelConfigBase:
    display_name = "ParallelConfig"

    def to_dict(self):
        return copy.deepcopy(self.__dict__)

    @classmethod
    def from_dict(cls, d):
        cfg = cls()
        for k, v in d.items():
            setattr(cfg, k, v)
        return cfg

    def _check_pipeline(self):
        pp = getattr(self, "pipeline_parallelism", 1)
        vpp = getattr(self, "virtual_pipeline_parallelism", 1)
        assert self.num_hidden_layers % pp == 0, (
            f"num_hidden_layers {self.num_hidden_layers} should be divisible by pipeline_parallelism {pp}")
        assert (self.num_hidden_layers // pp) % vpp == 0, (
            f"(num_hidden_layers / pipeline_parallelism) {self.num_hidden_layers // pp} should be divisible by "
            f"virtual_pipeline_parallelism {vpp}")

    def check_compatibility(self):
        self._check_pipeline()

    def __repr__(self):
        lines = [f"{self.display_name} : {{"]
        lines += [f'    "{k}": {v!r},' for k, v in self.__dict__.items()]
        lines.append("}")
        return "\n".join(lines)

    __str__ = __repr__
