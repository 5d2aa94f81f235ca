"""The path every generated token takes: ``DecodeRunner.step`` with captured CUDA
graphs (and programmatic dependent launch as the runner chooses), compared logit by
logit with the plain implementation, and in 32-bit bit by bit with the eager
``Engine.step`` of the same schedule.

A graph is keyed by the number of rows and by what the parts say changes their
launches (the attention's rounded longest length); everything else (which slots, which
positions, which pages) changes under the same key from step to step and from batch to
batch, so a replay that read a stale slot, position or page would show here as a wrong
logit, not only as a flipped argmax.
"""
import pytest
import torch

from helpers import SHARP, assert_close, make_model, plain_logits, random_prompts, reference_tensors

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _graphs_only(request):
    if request.config.getoption("--zlm-bounds-check"):
        pytest.skip("the bounds-check build runs without CUDA graphs")


DTYPES = ["float32", "bfloat16"]
NAMES = ["A", "B", "C"]


def build(tmp_path, name, dtype, max_tokens=2048, **kw):
    from zlm_b200 import Engine
    folder, cfg, tensors = make_model(tmp_path, name, seed=5, sharp=SHARP[dtype])
    eng = Engine.from_pretrained(folder, dtype=dtype, max_tokens=max_tokens, **kw)
    assert eng.decoder.use_graphs, "the decode runner must replay graphs by default"
    return eng, cfg, reference_tensors(tensors, dtype)


def greedy():
    from zlm_b200.sampling import SamplingParams
    return SamplingParams()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_graph_last_32_one_by_one(tmp_path, name, dtype):
    from zlm_b200 import StepEntry
    eng, cfg, ref = build(tmp_path, name, dtype)
    dec = eng.decoder
    n = min(cfg.max_position_embeddings, 150)
    (p,) = random_prompts(cfg.vocab_size, [n], seed=71)
    want = plain_logits(ref, cfg, p)
    s = eng.new_sequence()
    head = n - 32
    eng.step([StepEntry(s, p[:head], [])])
    got = []
    for t in range(head, n):
        dec.step([s], [p[t]], greedy())
        got.append(dec.last_logits[:1].clone())
    assert dec.replays > 0 and len(dec.graphs) < 32, "steps were not replayed from captured graphs"
    got = torch.cat(got)
    assert_close(got, want[head:], dtype, f"{name} last 32 through the graph")
    # the sampled token of the last step is the argmax of its logits
    assert int(dec.out[0]) == int(got[-1].argmax())
    eng.release(s)
    if dtype == "float32":
        # the same schedule through the eager step function: the same bits
        s = eng.new_sequence()
        eng.step([StepEntry(s, p[:head], [])])
        eager = torch.cat([eng.step([StepEntry(s, [p[t]], [0])]).clone() for t in range(head, n)])
        assert torch.equal(eager, got)
        eng.release(s)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_graph_unequal_batches_reuse_slots_under_one_key(tmp_path, name, dtype):
    """Unequal prompts decoded for different numbers of steps, so that rows end at
    different steps (4 -> 3 -> 2 rows ...) and the next batch takes the freed slots and
    pages; the batches have the same row counts and, at every step, a longest sequence of
    the same rounded size (the row that decodes 9 tokens is the one longer than a page), so
    the second and third batch replay the first batch's graphs with other slots, positions
    and pages."""
    from zlm_b200 import StepEntry
    eng, cfg, ref = build(tmp_path, name, dtype, max_tokens=64 * 8, max_batch=4)
    dec = eng.decoder
    cap = cfg.max_position_embeddings
    graphs_after_first = None
    for b in range(3):
        lens = [min(cap - 14, l) for l in ([3, 70, 17, 1], [30, 65, 2, 9], [20, 66, 1, 50])[b]]
        extra = [4, 9, 1, 12]
        full = random_prompts(cfg.vocab_size, [l + e for l, e in zip(lens, extra)], seed=80 + b)
        want = [plain_logits(ref, cfg, p) for p in full]
        slots = [eng.new_sequence() for _ in full]
        if b == 1:
            slots = slots[::-1]           # same slots as before, other rows in them
        eng.step([StepEntry(s, p[:l - 1], []) for s, p, l in zip(slots, full, lens) if l > 1])
        live = list(range(len(full)))
        eager_rows = []
        for step in range(-1, max(extra)):
            # step -1 feeds the last prompt token of every row through the graph path as well
            live = [j for j in live if step < extra[j]]
            for j in range(len(full)):
                if step == extra[j]:
                    eng.release(slots[j])
            toks = [full[j][lens[j] + step] for j in live]
            dec.step([slots[j] for j in live], toks, greedy())
            got = dec.last_logits[:len(live)].clone()
            eager_rows.append(([(j, lens[j] + step) for j in live], got))
            for r, j in enumerate(live):
                assert_close(got[r], want[j][lens[j] + step], dtype, f"{name} batch {b} row {j} step {step}")
        for j in range(len(full)):
            if extra[j] >= max(extra):
                eng.release(slots[j])
        eng.cache.check()
        if b == 0:
            graphs_after_first = len(dec.graphs)
        else:
            assert len(dec.graphs) == graphs_after_first, "a later batch captured graphs anew instead of replaying"
        if dtype == "float32" and b == 2:
            # the same schedule, eagerly through Engine.step: the same bits
            slots = [eng.new_sequence() for _ in full]
            eng.step([StepEntry(s, p[:l - 1], []) for s, p, l in zip(slots, full, lens) if l > 1])
            for rows, got in eager_rows:
                ents = [StepEntry(slots[j], [full[j][t]], [0]) for j, t in rows]
                assert torch.equal(eng.step(ents), got)
            for s in slots:
                eng.release(s)
    assert dec.replays > 0
    assert eng.cache.slots.held == 0 and all(g.pages.held == 0 for g in eng.cache.groups)


@pytest.mark.parametrize("dtype", DTYPES)
def test_graph_row_count_changes_and_comes_back(tmp_path, dtype):
    """4 rows, then 3 (one pauses), then 4 again with the paused row's slot given to a new
    sequence: the graph of 4 rows is replayed with a slot whose content is new."""
    from zlm_b200 import StepEntry
    eng, cfg, ref = build(tmp_path, "B", dtype, max_tokens=64 * 16, max_batch=4)
    dec = eng.decoder
    full = random_prompts(cfg.vocab_size, [40, 12, 33, 21, 18], seed=91)
    want = [plain_logits(ref, cfg, p) for p in full]
    fed = [8, 5, 9, 6, 7]                      # prompt tokens fed whole
    slots = [eng.new_sequence() for _ in range(4)]
    eng.step([StepEntry(slots[j], full[j][:fed[j]], []) for j in range(4)])
    pos = list(fed)
    rows = [0, 1, 2, 3]
    owner = {j: slots[j] for j in range(4)}

    def run(rs):
        dec.step([owner[j] for j in rs], [full[j][pos[j]] for j in rs], greedy())
        got = dec.last_logits[:len(rs)].clone()
        for r, j in enumerate(rs):
            assert_close(got[r], want[j][pos[j]], dtype, f"row {j} at {pos[j]}")
            pos[j] += 1

    for _ in range(3):
        run(rows)
    n4 = len(dec.graphs)
    for _ in range(3):
        run([0, 2, 3])                          # row 1 pauses
    eng.release(owner[1])                       # ... and ends; its slot goes to request 4
    owner[4] = eng.new_sequence()
    assert owner[4] == slots[1]
    eng.step([StepEntry(owner[4], full[4][:fed[4]], [])])
    before = len(dec.graphs)
    for _ in range(3):
        run([0, 4, 2, 3])
    assert len(dec.graphs) == before and n4 >= 1, "the 4-row graph was not replayed"
    assert dec.replays > 0


@pytest.mark.parametrize("rows", [8, 20, 30, 64])
def test_dependent_launches_change_no_bit(rows):
    """Decode steps with programmatic dependent launches and in plain stream order: the same
    kernels, so the same bits, at Qwen3-0.6B's layer sizes (two layers), where the steps of 20
    and 64 rows run the tcgen05 products with their shares and the split attention, and against
    the plain implementation for one of the rows.  At 30 rows the attention mixer asks for plain
    launches (one part per pair on about half the blocks the device holds); forced on, they still
    change nothing."""
    from zlm_b200 import Engine, StepEntry
    from zlm_b200.parts.model import DecoderModel
    from zlm_b200.registry import config_from_dict
    from zlm_b200.weights import random_tensors
    from zlm_b200.weights.loader import target_dtype
    from test_layer_sizes_gpu import SIZES, TOL_8B
    cfg = config_from_dict(dict(SIZES["0.6B"], vocab_size=2056))
    tensors = random_tensors(DecoderModel(cfg.to_model_spec()).param_specs(), 8, "cpu", torch.float32)
    specs = DecoderModel(cfg.to_model_spec()).param_specs()
    dev = {n: t.to("cuda").to(target_dtype(specs[n], t.dtype, torch.bfloat16)) for n, t in tensors.items()}
    eng = Engine(cfg, dev, torch.bfloat16, "cuda:0", max_tokens=rows * 512, max_batch=rows)
    dec = eng.decoder
    assert dec._pdl(rows) == (rows != 30)
    lens = [40 + (37 * i) % 300 for i in range(rows)]
    prompts = random_prompts(cfg.vocab_size, [n + 6 for n in lens], seed=88)
    runs = {}
    for pdl in (True, False):
        dec.use_pdl = pdl
        dec.graphs.clear()
        slots = [eng.new_sequence() for _ in range(rows)]
        eng.step([StepEntry(s, p[:n], []) for s, p, n in zip(slots, prompts, lens)])
        got = []
        for t in range(6):
            dec.step(slots, [p[n + t] for p, n in zip(prompts, lens)], greedy())
            got.append(dec.last_logits[:rows].clone())
        for s in slots:
            eng.release(s)
        runs[pdl] = torch.stack(got)
    assert torch.equal(runs[True], runs[False])
    want = plain_logits(reference_tensors(tensors, "bfloat16"), cfg, prompts[3][:lens[3] + 6])
    assert_close(runs[True][:, 3], want[lens[3]:], "bfloat16", f"row 3 of {rows}", TOL_8B["bfloat16"])
    assert eng.rt.k.status(sync=True) == 0
