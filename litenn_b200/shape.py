"""TensorShape and TensorAxes: validated, immutable, hashable shape / axes values with the
behaviour of litenn/core/TensorShape.py and litenn/core/TensorAxes.py (scalar shape ()
becomes (1,), negative axes need a rank, A+B concatenates, A-B removes, inversed())."""
from collections.abc import Iterable


class TensorAxes(Iterable):
    __slots__ = ["axes", "rank", "_inversed"]

    def __init__(self, axes, shape_rank=None):
        self._inversed = None
        if isinstance(axes, TensorAxes):
            self.axes, self.rank, self._inversed = axes.axes, axes.rank, axes._inversed
            return
        if axes is None:
            self.axes, self.rank = None, None
            return
        if not isinstance(axes, Iterable):
            axes = (axes,)
        out = []
        for x in axes:
            if x is None:
                raise ValueError(f"Incorrent value {x} in axes {axes}")
            x = int(x)
            if x < 0:
                if shape_rank is None:
                    raise ValueError(f"Incorrent value {x} in axes {axes}, or provide shape_rank")
                x += shape_rank
            if x in out:
                raise ValueError("Axes must contain unique values.")
            out.append(x)
        self.axes, self.rank = tuple(out), len(out)

    def is_none_axes(self):
        return self.axes is None

    def sorted(self):
        return TensorAxes(sorted(self.axes))

    def inversed(self):
        if self.is_none_axes():
            raise Exception("none-axes does not support inversed().")
        if self._inversed is None:
            pos = {axis: i for i, axis in enumerate(self.axes)}
            if sorted(pos) != list(range(self.rank)):
                raise Exception(f"axes {self.axes} are inconsistent to do inverse order.")
            self._inversed = TensorAxes([pos[i] for i in range(self.rank)])
        return self._inversed

    def __hash__(self):
        return hash(self.axes)

    def __eq__(self, other):
        if isinstance(other, TensorAxes):
            return self.axes == other.axes
        if isinstance(other, Iterable):
            return self.axes == tuple(other)
        return False

    def __iter__(self):
        if self.is_none_axes():
            raise Exception("none-axes does not support iteration.")
        return iter(self.axes)

    def __len__(self):
        return self.rank

    def __getitem__(self, key):
        if self.is_none_axes():
            raise Exception("none-axes does not support indexing.")
        if isinstance(key, slice):
            return TensorAxes(self.axes[key])
        return self.axes[key]

    def __add__(self, o):
        if not isinstance(o, Iterable):
            raise ValueError(f"unable to use type {o.__class__} in TensorAxes append")
        return TensorAxes(self.axes + tuple(o))

    def __radd__(self, o):
        if not isinstance(o, Iterable):
            raise ValueError(f"unable to use type {o.__class__} in TensorAxes append")
        return TensorAxes(tuple(o) + self.axes)

    def __sub__(self, o):
        if not isinstance(o, Iterable):
            raise ValueError(f"unable to use type {o.__class__} in TensorAxes substraction")
        drop = tuple(o)
        return TensorAxes([a for a in self.axes if a not in drop])

    def __rsub__(self, o):
        if not isinstance(o, Iterable):
            raise ValueError(f"unable to use type {o.__class__} in TensorAxes substraction")
        return TensorAxes([a for a in o if a not in self.axes])

    def __str__(self):
        return "(None)" if self.is_none_axes() else str(self.axes)

    def __repr__(self):
        return "TensorAxes" + str(self)


class TensorShape(Iterable):
    __slots__ = ["shape", "size", "rank"]

    def __init__(self, shape):
        if isinstance(shape, TensorShape):
            self.shape, self.size, self.rank = shape.shape, shape.size, shape.rank
            return
        if isinstance(shape, (int, float)):
            shape = (int(shape),)
        if not isinstance(shape, Iterable):
            raise ValueError("Invalid type to create TensorShape")
        dims, size = [], 1
        for x in shape:
            if x is None:
                raise ValueError(f"Incorrent value {x} in shape {shape}")
            x = int(x)
            if x < 1:
                raise ValueError(f"Incorrent value {x} in shape {shape}")
            dims.append(x)
            size *= x
        if not dims:
            dims = [1]       # scalar shape is stored as (1,)
        self.shape, self.rank, self.size = tuple(dims), len(dims), size

    def axes_arange(self):
        return TensorAxes(range(self.rank))

    def transpose_by_axes(self, axes):
        return TensorShape(self.shape[a] for a in TensorAxes(axes))

    def __hash__(self):
        return hash(self.shape)

    def __eq__(self, other):
        if isinstance(other, TensorShape):
            return self.shape == other.shape
        if isinstance(other, Iterable):
            return self.shape == tuple(other)
        return False

    def __iter__(self):
        return iter(self.shape)

    def __len__(self):
        return len(self.shape)

    def __getitem__(self, key):
        if isinstance(key, Iterable):
            if isinstance(key, TensorAxes) and key.is_none_axes():
                return self
            return self.transpose_by_axes(key)
        if isinstance(key, slice):
            return TensorShape(self.shape[key])
        return self.shape[key]

    def __add__(self, o):
        if not isinstance(o, Iterable):
            raise ValueError(f"unable to use type {o.__class__} in TensorShape append")
        return TensorShape(self.shape + tuple(o))

    def __radd__(self, o):
        if not isinstance(o, Iterable):
            raise ValueError(f"unable to use type {o.__class__} in TensorShape append")
        return TensorShape(tuple(o) + self.shape)

    def __str__(self):
        return str(self.shape)

    def __repr__(self):
        return "TensorShape" + str(self)
