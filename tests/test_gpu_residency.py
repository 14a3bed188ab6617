"""What a step moves between host and device, counted.

A step allocates no device memory, copies one buffer to the device (its index arrays, with the block-table
rows that changed and the sampler's counters inside) and one back (the sampled token ids with their status
words, 2 x rows integers).  The reference asserts the same of its CUDA path with counters of its own
(test/forward_test.cc:412-420: no host-to-device copy per token, one device-to-host copy).  Here the
counters are torch's allocator statistics and wrappers around the tensor methods that can move data."""
import pytest
import torch

import cpp_minilamma_b200 as ml
import tiny_configs as tc
from cpp_minilamma_b200 import EngineBackend, SamplingParams, StepEntry

pytestmark = pytest.mark.gpu


class Traffic:
    """Counts, while active, copies by direction (h2d, d2h, d2d; with the number of elements of each) and
    requests to the device allocator."""

    MOVERS = ("cpu", "tolist", "item", "numpy", "to", "cuda", "clone", "contiguous")

    def __enter__(self):
        self.copies = {"h2d": [], "d2h": [], "d2d": []}
        self.other = []
        self._saved = {name: getattr(torch.Tensor, name) for name in ("copy_",) + self.MOVERS}
        traffic = self

        def copy_(dst, src, *args, **kwargs):
            kind = {("cpu", "cuda"): "h2d", ("cuda", "cpu"): "d2h", ("cuda", "cuda"): "d2d"}.get(
                (src.device.type, dst.device.type))
            if kind:
                traffic.copies[kind].append(dst.numel())
            return traffic._saved["copy_"](dst, src, *args, **kwargs)

        torch.Tensor.copy_ = copy_
        for name in self.MOVERS:
            def wrapped(tensor, *args, _name=name, **kwargs):
                if tensor.is_cuda:
                    traffic.other.append(_name)
                return traffic._saved[_name](tensor, *args, **kwargs)
            setattr(torch.Tensor, name, wrapped)
        torch.cuda.synchronize()
        self._allocated = torch.cuda.memory_stats()["allocation.all.allocated"]
        return self

    def __exit__(self, *exc):
        torch.cuda.synchronize()
        self.allocations = torch.cuda.memory_stats()["allocation.all.allocated"] - self._allocated
        for name, method in self._saved.items():
            setattr(torch.Tensor, name, method)
        return False

    def expect_one_in_one_out(self, rows, what):
        assert self.allocations == 0, f"{what}: {self.allocations} device allocations"
        assert len(self.copies["h2d"]) == 1, f"{what}: host-to-device copies {self.copies['h2d']}"
        assert self.copies["d2h"] == [2 * rows], f"{what}: device-to-host copies {self.copies['d2h']}"
        assert not self.other, f"{what}: device tensors were moved or cloned by {self.other}"


@pytest.mark.parametrize("name,dtype", [("D", "bfloat16"), ("B", "float32")])
@pytest.mark.parametrize("sampling", [SamplingParams(), SamplingParams(temperature=0.8, top_k=10, seed=4)])
@pytest.mark.parametrize("use_graphs", [True, False])
def test_a_decode_step_allocates_nothing_and_copies_one_buffer_each_way(model_folders, name, dtype, sampling, use_graphs):
    llm = ml.load(model_folders(name, dtype), dtype=dtype, max_tokens=4096, max_seqs=4)
    backend = EngineBackend(llm.engine, sampling, use_graphs=use_graphs)
    rows = backend.sampler.rows
    prompts = [tc.random_tokens(name, n, 40 + n) for n in (60, 3, 17)]
    slots = backend.acquire(3)
    requests = [0, 1, 2]

    def prompt_step():
        entries = [StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)]
        return backend.collect(backend.submit(entries, requests, [0, 0, 0]))

    last = prompt_step()
    for s in slots:      # the same prompts again: the workspace has its sizes now
        backend.release(s)
    slots = backend.acquire(3)
    with Traffic() as traffic:
        last = prompt_step()
    traffic.expect_one_in_one_out(rows, "prompt step")
    crossed = False
    for step in range(1, 12):
        entries = [StepEntry(s, [t], [0]) for s, t in zip(slots, last)]
        before = [len(llm.engine.cache.groups[0].pages[s]) for s in slots]
        with Traffic() as traffic:
            last = backend.collect(backend.submit(entries, requests, [step] * 3))
        crossed = crossed or before != [len(llm.engine.cache.groups[0].pages[s]) for s in slots]
        if step >= 3:  # the first decode step runs eagerly and sizes the workspace, the second is captured
            traffic.expect_one_in_one_out(rows, f"decode step {step}")
    assert crossed, "no sequence crossed a page: the block-table rows were never sent"
    if use_graphs:
        assert backend.graphs.replays >= 8
        # a step ahead of the host takes its tokens on the device (a gather kernel, by the previous step's rows):
        # no further copy; it may leave out sequences that ended with the step before
        from cpp_minilamma_b200.csrc import kernels as K
        backend.submit([StepEntry(s, [t], [0]) for s, t in zip(slots, last)], requests, [12] * 3)
        gathers = K.calls.get("gather_int32", 0)
        with Traffic() as traffic:
            ticket = backend.submit_ahead(slots, requests, [13] * 3)
        assert traffic.allocations == 0 and len(traffic.copies["h2d"]) == 1 and traffic.copies["d2d"] == []
        assert K.calls.get("gather_int32", 0) == gathers + 1
        backend.collect(ticket)
        with Traffic() as traffic:
            ticket = backend.submit_ahead([slots[2], slots[0]], [2, 0], [14] * 2)
        assert len(traffic.copies["h2d"]) == 1 and traffic.copies["d2d"] == []
        assert len(backend.collect(ticket)) == 2
        with pytest.raises(ValueError, match="did not have"):
            backend.submit_ahead([slots[1]], [1], [15])
    for s in slots:
        backend.release(s)
    llm.engine.cache.check()
