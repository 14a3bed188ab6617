"""What the host does when a kernel reports that it gave up (a bounded wait that ran out).

No kernel has to fail for these tests: the flags are set from the host (`raise_device_error`), or the
status words that the sampler reads are written by hand."""
import pytest
import torch

from cpp_minilamma_b200.csrc.kernels import DeviceKernelError
from cpp_minilamma_b200.sampling.sampler import DeviceSampler


class _Done:
    def synchronize(self):
        pass


def _host_only_sampler(rows):
    sampler = DeviceSampler.__new__(DeviceSampler)  # without its device buffers: `collect` reads host memory only
    sampler.rows = rows
    sampler.hosts = [torch.zeros(2 * rows, dtype=torch.int32) for _ in range(2)]
    sampler.events = [_Done(), _Done()]
    return sampler


def test_collect_reads_tokens_error_bits_and_the_non_finite_mark():
    sampler = _host_only_sampler(4)
    sampler.hosts[1][:3] = torch.tensor([7, 8, 9], dtype=torch.int32)
    assert sampler.collect((1, 3, 4)) == [7, 8, 9]
    sampler.hosts[1][4] = 0x400  # bit 2 of the error flags, carried in bits 8 and up of row 0's status word
    with pytest.raises(DeviceKernelError, match="tcgen05 prefill attention"):
        sampler.collect((1, 3, 4))
    sampler.hosts[1][4] = 0x900
    with pytest.raises(DeviceKernelError, match="TMA linear kernel.*TMA decode attention"):
        sampler.collect((1, 3, 4))
    sampler.hosts[1][4] = 0
    sampler.hosts[1][6] = 1      # row 2 saw a logit that is not finite
    with pytest.raises(FloatingPointError):
        sampler.collect((1, 3, 4))
    assert sampler.collect((1, 2, 4)) == [7, 8]  # rows beyond the ticket's count are not looked at


@pytest.mark.gpu
def test_flags_set_from_the_host_are_read_once():
    from cpp_minilamma_b200.csrc import kernels as K
    torch.zeros(1, device="cuda:0")
    assert K.take_device_error() == 0
    K.raise_device_error(0b0101)
    assert K.take_device_error() == 0b0101
    assert K.take_device_error() == 0
    with pytest.raises(K.KernelError):
        K.raise_device_error(16)


@pytest.mark.gpu
@pytest.mark.parametrize("mask", [1, 2, 4, 8])
def test_generation_and_step_raise_and_recover(model_folders, mask):
    import cpp_minilamma_b200 as ml
    from cpp_minilamma_b200 import StepEntry
    from cpp_minilamma_b200.csrc import kernels as K
    llm = ml.load(model_folders("D", "bfloat16"), dtype="bfloat16", max_tokens=2048)
    prompts = [[5, 17, 3, 200, 9] * 20, [1, 2]]
    clean = llm.generate(prompts, max_new_tokens=12, ignore_eos=True)
    assert llm.engine.shared_decode_graphs().replays > 0
    K.raise_device_error(mask)
    with pytest.raises(DeviceKernelError, match=K.DEVICE_ERROR_BITS[mask.bit_length() - 1]):
        llm.generate(prompts, max_new_tokens=12, ignore_eos=True)
    assert not llm.engine.shared_decode_graphs()._captured      # the graphs were dropped
    assert llm.engine.cache.n_free_slots == llm.engine.cache.n_slots
    assert llm.generate(prompts, max_new_tokens=12, ignore_eos=True) == clean
    # the step function reports it too, at the place where its caller would read the logits
    slot, = llm.engine.acquire(1)
    K.raise_device_error(mask)
    with pytest.raises(DeviceKernelError):
        llm.engine.step([StepEntry(slot, [1, 2, 3], [2])])
    again = llm.engine.step([StepEntry(slot, [4], [0])])
    assert torch.isfinite(again).all()
    llm.engine.release(slot)
    assert K.take_device_error() == 0
