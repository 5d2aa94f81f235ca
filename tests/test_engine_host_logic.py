"""The engine's host logic (step planning, paging, windows, slot reuse, errors)
on a machine without a GPU: the CUDA library is replaced by the plain torch
stand-ins of tests/cpu_kernels.py, everything else is the product's code."""
import pytest
import torch

from cpu_kernels import PlainKernels
from helpers import plain_logits, random_prompts
from tiny_configs import TINY
from zlm_b200 import Engine, StepEntry, StepError
from zlm_b200.cache import CacheFull
from zlm_b200.parts.model import DecoderModel
from zlm_b200.registry import config_from_dict
from zlm_b200.weights import random_tensors


def build(name, **kw):
    cfg = config_from_dict(TINY[name])
    t = random_tensors(DecoderModel(cfg.to_model_spec()).param_specs(), 2)
    kw.setdefault("max_tokens", 1024)
    return Engine(cfg, dict(t), torch.float32, "cpu", kernels=PlainKernels(), **kw), cfg, t


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_cuttings_agree_with_the_plain_implementation(name):
    eng, cfg, t = build(name)
    ps = random_prompts(cfg.vocab_size, [70, 9, 33], seed=1)
    want = [plain_logits(t, cfg, p) for p in ps]
    slots = [eng.new_sequence() for _ in ps]
    cut = [40, 4, 20]
    got = eng.step([StepEntry(s, p[:c], list(range(c))) for s, p, c in zip(slots, ps, cut)]).clone()
    off = 0
    for p, w, c in zip(ps, want, cut):
        assert float((got[off:off + c] - w[:c]).abs().max()) < 1e-5
        off += c
    for i in range(5):       # rows go on one by one; the shortest leaves first
        ents = [(j, StepEntry(slots[j], [ps[j][cut[j] + i]], [0])) for j in range(3) if cut[j] + i < len(ps[j])]
        got = eng.step([e for _, e in ents]).clone()
        for r, (j, _) in enumerate(ents):
            assert float((got[r] - want[j][cut[j] + i]).abs().max()) < 1e-5
    for s in slots:
        eng.release(s)
    eng.cache.check()
    assert eng.cache.slots.held == 0


def test_step_errors_come_before_any_work():
    eng, cfg, _ = build("A", max_tokens=128, max_batch=2)
    s = eng.new_sequence()
    with pytest.raises(StepError, match="outside the vocabulary"):
        eng.step([StepEntry(s, [1, cfg.vocab_size], [])])
    with pytest.raises(StepError, match="appears twice"):
        eng.step([StepEntry(s, [1], []), StepEntry(s, [2], [])])
    with pytest.raises(StepError, match="not held"):
        eng.step([StepEntry(1, [1], [])])
    with pytest.raises(StepError, match="wanted place 3"):
        eng.step([StepEntry(s, [1, 2], [3])])
    with pytest.raises(StepError, match="no token"):
        eng.step([StepEntry(s, [], [])])
    with pytest.raises(StepError, match="at least one"):
        eng.step([])
    assert eng.length(s) == 0 and eng.steps_run == 0
    eng.step([StepEntry(s, [1] * 100, [])])
    with pytest.raises(CacheFull):
        eng.step([StepEntry(s, [1] * 29, [])])       # 129 tokens need a third page; there are two
    assert eng.length(s) == 100
    assert eng.step([StepEntry(s, [1] * 28, [])]) is None


def test_schedule_may_repeat_a_layer_and_share_a_cache():
    """A model whose schedule runs layer 0 twice (weights shared, a cache each) and
    whose last entry reads entry 1's cache instead of writing one."""
    from dataclasses import replace
    from zlm_b200.config import ScheduleEntry
    cfg = config_from_dict(TINY["A"])
    spec = cfg.to_model_spec()
    sched = (ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0), ScheduleEntry(1, cache_of=1))

    class Cfg2:
        eos_token_ids = ()
        def to_model_spec(self):
            return replace(spec, schedule=sched)

    t = random_tensors(DecoderModel(spec).param_specs(), 4)
    eng = Engine(Cfg2(), dict(t), torch.float32, "cpu", max_tokens=256, kernels=PlainKernels())
    assert len(eng.cache.groups) == 1 and eng.cache.groups[0].entries == [0, 1, 2]
    (p,) = random_prompts(cfg.vocab_size, [20], seed=3)
    s = eng.new_sequence()
    whole = eng.step([StepEntry(s, p, list(range(20)))]).clone()
    eng.release(s)
    s = eng.new_sequence()
    parts = [eng.step([StepEntry(s, p[:13], list(range(13)))]).clone()]
    parts += [eng.step([StepEntry(s, [p[i]], [0])]).clone() for i in range(13, 20)]
    assert float((torch.cat(parts) - whole).abs().max()) < 1e-5
    # and it is not the plain two-layer model
    assert float((whole - plain_logits(t, cfg, p)).abs().max()) > 1e-3


def test_a_place_named_twice_is_refused():
    eng, cfg, _ = build("A", max_tokens=128, max_batch=2, max_step_tokens=4)
    s = eng.new_sequence()
    with pytest.raises(StepError, match="may be named once"):
        eng.step([StepEntry(s, [1, 2], [0, 1, 1])])
    assert eng.length(s) == 0


class ReportingKernels(PlainKernels):
    """Plain kernels with the CUDA library's status word: ``pending`` stands for a mark that
    a kernel's bounded wait left there."""
    pending = 0

    def check_status(self, sync=False):
        from zlm_b200.kernels import KernelError
        if self.pending:
            code, self.pending = self.pending, 0
            raise KernelError(f"a bounded wait inside a kernel gave up (status {code:#x})")


def test_a_reported_give_up_raises_where_the_host_waits_anyway():
    from zlm_b200.kernels import KernelError
    cfg = config_from_dict(TINY["A"])
    t = random_tensors(DecoderModel(cfg.to_model_spec()).param_specs(), 2)
    k = ReportingKernels()
    eng = Engine(cfg, dict(t), torch.float32, "cpu", kernels=k, max_tokens=512)
    assert len(eng.generate([[1, 2, 3], [4, 5]], max_tokens=3).tokens[0]) == 3
    # reported during a prefill: generate raises, and gives its slots back
    k.pending = 0x102
    with pytest.raises(KernelError, match="gave up"):
        eng.generate([[1, 2, 3], [4, 5]], max_tokens=3)
    assert eng.cache.slots.held == 0
    # reported during a decode step: the fetch of that step raises
    s = eng.new_sequence()
    eng.step([StepEntry(s, [1, 2, 3], [])])
    k.pending = 0x203
    from zlm_b200.sampling import SamplingParams
    h = eng.decode_launch([s], [4], SamplingParams(), [0])
    with pytest.raises(KernelError, match="0x203"):
        eng.decode_fetch(h)
    # reported by a step whose logits the caller has not read yet: the next step says so
    k.pending = 0x101
    with pytest.raises(KernelError, match="0x101"):
        eng.step([StepEntry(s, [5], [0])])
    assert eng.step([StepEntry(s, [5], [0])] ) is not None
    eng.release(s)


def test_tensors_can_be_read_back_by_their_checkpoint_names():
    eng, cfg, t = build("B")
    names = eng.model.tensor_names()
    assert set(names) == set(t)
    for n in names:
        assert torch.equal(eng.tensor(n).float(), t[n].float()), n
    with pytest.raises(KeyError, match="no tensor"):
        eng.tensor("model.layers.99.mlp.up_proj.weight")
    tied, cfg_a, ta = build("A")
    assert torch.equal(tied.tensor("lm_head.weight"), ta["model.embed_tokens.weight"])


def test_a_width_that_no_bf16_kernel_takes_is_refused_when_the_model_is_built():
    from zlm_b200.kernels import CudaKernels, KernelError
    w = torch.zeros((16, 36), dtype=torch.bfloat16)
    with pytest.raises(KernelError, match=r"SwiGLU.down_proj \[16, 36\].*multiple of 8"):
        CudaKernels.check_linear(None, "SwiGLU.down_proj", w)
    CudaKernels.check_linear(None, "x", torch.zeros((16, 36)))            # 32-bit: any width
    CudaKernels.check_linear(None, "x", torch.zeros((16, 40), dtype=torch.bfloat16))
