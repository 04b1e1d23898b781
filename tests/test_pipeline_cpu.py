"""Host logic of PipelinedSampler without a GPU: the order of submit() / next() calls it makes on the
pipeline object (how far it runs ahead, that it drains, that nothing is reordered), and the registration of
torch.classes.dgs_classes.BlockPipeline with the methods the wrapper calls."""
import pytest
import torch  # noqa: F401  (the annotations of _drive are resolved in this module)


class FakePipe:
    """Stands in for torch.classes.dgs_classes.BlockPipeline: records the calls, enforces the slot rule."""

    def __init__(self, depth):
        self.depth, self.queue, self.log = depth, [], []

    def submit(self, seeds):
        assert len(self.queue) < self.depth, "submitted into a full pipeline"
        self.queue.append(seeds)
        self.log.append(("submit", seeds))

    def next(self):
        assert self.queue, "next() on an empty pipeline"
        seeds = self.queue.pop(0)
        self.log.append(("next", seeds))
        rows = [[seeds] * 2, [seeds] * 3]                 # two "blocks" with 2 and 3 edges
        return ("frontier%d" % seeds, [_T(r) for r in rows], [_T(r) for r in rows], [5, 4, 4, 1], "x%d" % seeds)


class _T(list):
    def numel(self):
        return len(self)


@pytest.mark.parametrize("depth,n_batches", [(1, 4), (3, 7), (4, 2), (6, 0)])
def test_generator_runs_depth_ahead_and_drains(pkg, depth, n_batches):
    s = pkg.PipelinedSampler.__new__(pkg.PipelinedSampler)
    s.depth, s.pipe = depth, FakePipe(depth)
    got = list(s(range(n_batches)))
    assert [g[0] for g in got] == ["frontier%d" % i for i in range(n_batches)]          # in order, none lost
    assert all(g[2] == 5 and g[3] == "x%d" % i for i, g in enumerate(got))              # n_edges = 2 + 3
    assert got == [] or got[0][1] == [([0, 0], [0, 0], 5, 4), ([0, 0, 0], [0, 0, 0], 4, 1)]
    assert not s.pipe.queue                                                             # drained
    # the first next() comes after min(depth, n) submits; from then on they alternate
    log = s.pipe.log
    first_next = next((i for i, e in enumerate(log) if e[0] == "next"), len(log))
    assert first_next == min(depth, n_batches)
    in_flight = peak = 0
    for kind, _ in log:
        in_flight += 1 if kind == "submit" else -1
        peak = max(peak, in_flight)
    assert peak == min(depth, n_batches)


def _drive(p: "torch.classes.dgs_classes.BlockPipeline", s: "torch.Tensor"):
    p.submit(s)
    n = p.pending() + p.depth()
    return p.next(), n


def test_block_pipeline_class_is_registered_with_the_methods_the_wrapper_calls(pkg):
    """TorchScript compiles a function that calls every method (no instance, so no GPU needed): a missing
    method or a changed signature fails here."""
    import torch
    pkg.load_ops()
    g = torch.jit.script(_drive)
    text = str(g.graph)
    for m in ("submit", "pending", "depth", "next"):
        assert 'name="%s"' % m in text
    assert "(Tensor, Tensor[], Tensor[], int[], Tensor)" in text          # what next() returns
