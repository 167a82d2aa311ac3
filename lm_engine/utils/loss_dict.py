from __future__ import annotations


class MetricsTrackingDict:
    """Small numeric dict supporting ``+`` and ``/`` with a dict/tracker (key-wise) or a scalar; prints one ``key = value`` line per entry
    (parity: lm_engine/utils/loss_dict.py:8-59)."""

    def __init__(self, data: dict | None = None) -> None:
        self.data = dict(data or {})

    def __getitem__(self, key):
        return self.data[key]

    def __setitem__(self, key, value) -> None:
        self.data[key] = value

    def __contains__(self, key) -> bool:
        return key in self.data

    def __iter__(self):
        return iter(self.data)

    def __len__(self) -> int:
        return len(self.data)

    def keys(self):
        return self.data.keys()

    def values(self):
        return self.data.values()

    def items(self):
        return self.data.items()

    def get_dict(self) -> dict:
        return self.data

    def _combine(self, other, op):
        if isinstance(other, MetricsTrackingDict):
            other = other.data
        if isinstance(other, dict):
            for key, value in other.items():
                self.data[key] = op(self.data[key], value) if key in self.data else value
        else:
            for key in self.data:
                self.data[key] = op(self.data[key], other)
        return self

    def __add__(self, other):
        return self._combine(other, lambda a, b: a + b)

    __iadd__ = __add__

    def __truediv__(self, other):
        if isinstance(other, MetricsTrackingDict):
            other = other.data
        if isinstance(other, dict):  # key-wise; a key that is only in the divisor starts from zero
            for key, value in other.items():
                self.data[key] = self.data.get(key, 0) / value
            return self
        for key in self.data:
            self.data[key] = self.data[key] / other
        return self

    __itruediv__ = __truediv__

    def __repr__(self) -> str:
        return "\n".join(f"{key} = {value}" for key, value in self.data.items())
