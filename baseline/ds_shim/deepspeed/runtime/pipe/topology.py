"""Cartesian rank topology (axes pipe x data x model, model fastest-varying)."""
import collections
import itertools


class ProcessTopology:
    def __init__(self, axes, dims):
        self.axes, self.dims = list(axes), list(dims)
        self.Coord = collections.namedtuple("ProcessCoord", self.axes)
        self._rank_of = {}
        for r, c in enumerate(itertools.product(*[range(d) for d in self.dims])):
            self._rank_of[self.Coord(*c)] = r
        self._coord_of = {r: c for c, r in self._rank_of.items()}

    def get_axis_names(self):
        return list(self.axes)

    def get_dim(self, axis):
        return self.dims[self.axes.index(axis)] if axis in self.axes else 0

    def world_size(self):
        return len(self._rank_of)

    def get_coord(self, rank):
        return self._coord_of[rank]

    def get_rank(self, **coords):
        return self._rank_of[self.Coord(**coords)]

    def filter_match(self, **fixed):
        return sorted(r for c, r in self._rank_of.items() if all(getattr(c, k) == v for k, v in fixed.items()))

    def get_axis_list(self, axis, idx):
        return self.filter_match(**{axis: idx})

    def get_axis_comm_lists(self, axis):
        if axis not in self.axes:
            return []
        others = [a for a in self.axes if a != axis]
        out = []
        for c in itertools.product(*[range(self.get_dim(a)) for a in others]):
            fixed = dict(zip(others, c))
            out.append([self.get_rank(**fixed, **{axis: i}) for i in range(self.get_dim(axis))])
        return out

    def get_rank_repr(self, rank, omit_axes=("data", "pipe"), inner_sep="_", outer_sep="-"):
        c = self.get_coord(rank)
        return outer_sep.join(f"{a}{inner_sep}{getattr(c, a):02d}" for a in self.axes if a not in omit_axes)

    def __str__(self):
        return str(self._rank_of)


class PipeModelDataParallelTopology(ProcessTopology):
    def __init__(self, num_pp, num_mp, num_dp):
        super().__init__(axes=["pipe", "data", "model"], dims=[num_pp, num_dp, num_mp])


class PipeDataParallelTopology(ProcessTopology):
    def __init__(self, num_pp, num_dp):
        super().__init__(axes=["pipe", "data"], dims=[num_pp, num_dp])
