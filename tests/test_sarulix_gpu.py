"""Sarulix through the engine against the plain implementation (tests/plain/sarulix_plain.py, float64 on the CPU):
whole prompts, portions, token by token, batches, pages and state slots used again, graphs replayed, generation."""
import pytest
import torch

from tests import sarulix_util as su

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["MIXED", "WIDE", "ODD"])
def test_whole_prompt_and_portions_match_the_plain_model(name, dtype):
    cfg = getattr(su, name)
    model, tensors = su.build(cfg, seed=3, dtype=dtype)
    ids = su.ids_for(cfg, 75, seed=1)
    want = su.plain_logits(cfg, tensors, ids)
    drv = su.driver(model, dtype)
    su.assert_close(su.run_in_portions(drv, "a", ids, [len(ids)]), want, dtype)
    su.assert_close(su.run_in_portions(drv, "a", ids, [33, 2, 1, 17, 1]), want, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_portions_of_any_size_and_single_tokens_give_the_whole_prompts_logits(dtype):
    cfg = su.MIXED
    model, tensors = su.build(cfg, seed=4, dtype=dtype)
    ids = su.ids_for(cfg, 101, seed=2)
    want = su.plain_logits(cfg, tensors, ids)
    drv = su.driver(model, dtype)
    for portions in ([1], [2], [3, 2, 33, 31, 1, 16, 2], [32, 32, 5, 1], [47, 1, 1, 2]):
        got = su.run_in_portions(drv, "a", ids, portions)
        su.assert_close(got, want, dtype, portions)
    assert drv.executor.cache.all_free()


@pytest.mark.parametrize("eager", [True, False])
@pytest.mark.parametrize("dtype", DTYPES)
def test_prompts_that_cross_tiles_of_the_tensor_core_attention(dtype, eager):
    """300 tokens whole, in portions whose tiles of 64 queries begin anywhere among the keys' tiles, and beside another
    request; launched and replayed."""
    cfg = su.TENSOR
    model, tensors = su.build(cfg, seed=15, dtype=dtype)
    ids, other = su.ids_for(cfg, 300, seed=5), su.ids_for(cfg, 90, seed=6)
    want, want_other = su.plain_logits(cfg, tensors, ids), su.plain_logits(cfg, tensors, other)
    drv = su.driver(model, dtype, pool_tokens=448, eager=eager)
    su.assert_close(su.run_in_portions(drv, "a", ids, [300]), want, dtype)
    su.assert_close(su.run_in_portions(drv, "a", ids, [130, 70, 1, 2, 97]), want, dtype)
    got_a = [drv.step([("a", ids[:200], list(range(200)))])]
    out = drv.step([("a", ids[200:], list(range(100))), ("b", other, list(range(90)))], end=["a", "b"])
    su.assert_close(torch.cat([got_a[0], out[:100]]), want, dtype)
    su.assert_close(out[100:], want_other, dtype)


def test_the_logits_do_not_depend_on_the_cut_beyond_rounding():
    """float32: token by token, in twos and whole agree far inside the tolerance against the plain model."""
    cfg = su.WIDE
    model, _ = su.build(cfg, seed=14, dtype="float32")
    ids = su.ids_for(cfg, 60, seed=3)
    drv = su.driver(model, "float32")
    whole = su.run_in_portions(drv, "a", ids, [60])
    for portions in ([1], [2], [17, 3]):
        assert su.relative_error(su.run_in_portions(drv, "a", ids, portions), whole) < 2e-6, portions


@pytest.mark.parametrize("eager", [True, False])
@pytest.mark.parametrize("dtype", DTYPES)
def test_unequal_requests_in_one_batch_match_each_alone(dtype, eager):
    """Three requests of different lengths, portions of some beside single tokens of others; launched kernel by kernel and
    replayed from the graphs of the steps' shapes."""
    cfg = su.MIXED
    model, tensors = su.build(cfg, seed=5, dtype=dtype)
    ids = {"a": su.ids_for(cfg, 70, 11), "b": su.ids_for(cfg, 19, 12), "c": su.ids_for(cfg, 41, 13)}
    want = {r: su.plain_logits(cfg, tensors, t) for r, t in ids.items()}
    drv = su.driver(model, dtype, eager=eager)
    plan = {"a": [33, 1, 1, 2, 30, 1, 1, 1], "b": [2, 1, 1, 1, 14], "c": [1, 1, 17, 2, 20]}
    pos = {r: 0 for r in ids}
    got = {r: [] for r in ids}
    k = 0
    while any(pos[r] < len(ids[r]) for r in ids):
        entries, owners, end = [], [], []
        for r in ids:
            if pos[r] >= len(ids[r]) or (r == "b" and k == 2):          # b sits one step out
                continue
            n = min(plan[r][min(k, len(plan[r]) - 1)], len(ids[r]) - pos[r])
            entries.append((r, ids[r][pos[r]:pos[r] + n], list(range(n))))
            owners.append((r, n))
            pos[r] += n
            if pos[r] == len(ids[r]):
                end.append(r)
        out = drv.step(entries, end=end)
        at = 0
        for r, n in owners:
            got[r].append(out[at:at + n])
            at += n
        k += 1
    for r in ids:
        su.assert_close(torch.cat(got[r]), want[r], dtype, r)
    if not eager:
        assert drv.executor.n_shaped_steps > 0


@pytest.mark.parametrize("dtype", DTYPES)
def test_pages_and_state_slots_are_used_again(dtype):
    """A pool of 6 pages and 2 state slots, five requests one after and beside another: every page and slot serves
    several requests, and a request that starts in a used slot starts from an empty state and an empty convolution."""
    cfg = su.MIXED
    model, tensors = su.build(cfg, seed=6, dtype=dtype)
    drv = su.driver(model, dtype, pool_tokens=96, page_size=16, max_num_seqs=2)
    lengths = [40, 50, 33, 17, 48]
    all_ids = [su.ids_for(cfg, n, 20 + i) for i, n in enumerate(lengths)]
    want = [su.plain_logits(cfg, tensors, t) for t in all_ids]
    slots_seen = set()
    got0 = su.run_in_portions(drv, 0, all_ids[0], [13, 27])
    su.assert_close(got0, want[0], dtype)
    for a, b in ((1, 2), (3, 4)):
        ga, gb = [], []
        pa = pb = 0
        while pa < lengths[a] or pb < lengths[b]:
            entries = []
            na = min(11, lengths[a] - pa)
            nb = min(20 if pb == 0 else 1, lengths[b] - pb)
            if na:
                entries.append((a, all_ids[a][pa:pa + na], list(range(na))))
            if nb:
                entries.append((b, all_ids[b][pb:pb + nb], list(range(nb))))
            pa, pb = pa + na, pb + nb
            end = [r for r, p, n in ((a, pa, na), (b, pb, nb)) if n and p == lengths[r]]
            out = drv.step(entries, end=[])
            slots_seen |= {drv.executor.cache.state.slot(r) for r, _, _ in entries}
            for r in end:
                drv.executor.release(r)
                del drv.positions[r]
            if na:
                ga.append(out[:na])
            if nb:
                gb.append(out[na:na + nb])
        su.assert_close(torch.cat(ga), want[a], dtype, a)
        su.assert_close(torch.cat(gb), want[b], dtype, b)
    assert slots_seen == {0, 1}
    assert drv.executor.cache.all_free()


@pytest.mark.parametrize("needle_at", [0, 3, 15, 16, 17, 255, 256, 298])
def test_one_key_decides_wherever_it_lies(needle_at):
    """The last token's query finds the key of one token only (`plant_needle`): far back, the first of the sequence, on
    either side of a page's border (pages of 16), the newest but one; in a whole prompt, in portions cut at and beside
    the needle, and with the probe decoded alone after single tokens.  Without the needle the oracle's own last row
    moves by hundreds of tolerances, so a key or value taken from the wrong place could not hide."""
    cfg = su.NEEDLE
    model, tensors = su.build(cfg, seed=7, dtype="float32", sigma=0.3, prepare=su.plant_needle)
    n = 300
    ids = su.needle_ids(cfg, n, needle_at, 31)
    want = su.plain_logits(cfg, tensors, ids)
    without = list(ids)
    without[needle_at] = su.FILLER_ID
    assert su.relative_error(su.plain_logits(cfg, tensors, without)[-1:], want[-1:]) > 300 * su.TOL["float32"]
    drv = su.driver(model, "float32", pool_tokens=320)
    cut = max(needle_at, 1)
    for portions in ([n], [cut, 1, 2, n], [needle_at + 1, 1, n], [290] + [1] * 10):
        got = su.run_in_portions(drv, "a", ids, portions)
        assert su.relative_error(got, want) < su.TOL["float32"], portions


@pytest.mark.parametrize("name", ["KEEPING_LRU", "KEEPING_DELTA"])
def test_a_state_that_forgets_little_is_carried_through_portions_and_long_decoding(name):
    cfg = getattr(su, name)
    model, tensors = su.build(cfg, seed=8, dtype="float32", prepare=su.keep_long)
    ids = su.ids_for(cfg, 400, 41)
    want = su.plain_logits(cfg, tensors, ids)
    drv = su.driver(model, "float32", pool_tokens=448)
    for portions in ([400], [31, 33, 32, 1, 2, 64, 1], [100] + [1] * 300):
        got = su.run_in_portions(drv, "a", ids, portions)
        assert su.relative_error(got, want) < su.TOL["float32"], portions[:3]
    # a state lost where a portion was cut would show at the next token: the plain model started there differs
    for cut in (31, 100, 398):
        restarted = su.plain_logits(cfg, tensors, ids[cut:cut + 2])
        assert su.relative_error(restarted[:1], want[cut:cut + 1]) > 100 * su.TOL["float32"], cut
    if name == "KEEPING_LRU":
        # and the first token still counts at the end: without it the last logits differ
        shifted = su.plain_logits(cfg, tensors, ids[1:])
        assert su.relative_error(shifted[-1:], want[-1:]) > 30 * su.TOL["float32"]


@pytest.mark.parametrize("name", ["MIXED", "ODD"])
def test_the_first_tokens_of_a_sequence(name):
    """One, two and three tokens: the convolutions read zeros before the start, the sink outweighs a lone key, the
    recurrences start from nothing."""
    cfg = getattr(su, name)
    model, tensors = su.build(cfg, seed=9, dtype="float32")
    drv = su.driver(model, "float32")
    for n in (1, 2, 3, 6):
        ids = su.ids_for(cfg, n, 50 + n)
        for portions in ([1], [n]):
            got = su.run_in_portions(drv, "a", ids, portions)
            assert su.relative_error(got, su.plain_logits(cfg, tensors, ids)) < su.TOL["float32"], (n, portions)


@pytest.mark.parametrize("eager", [True, False])
def test_greedy_generation_through_the_engine_and_its_scheduler(eager):
    """`LLM.generate` (scheduler, chunked prompts, decode graphs, sampling kernel) against greedy decoding with the
    plain model."""
    from llmgen_b200.engine.api import LLM
    from llmgen_b200.sampling.params import SamplingParams
    cfg = su.MIXED
    model, tensors = su.build(cfg, seed=10, dtype="float32")
    prompts = [su.ids_for(cfg, n, 60 + n) for n in (9, 21, 4)]
    new = 10
    ref = []
    for p in prompts:
        seq = list(p)
        for _ in range(new):
            seq.append(int(su.plain_logits(cfg, tensors, seq)[-1].argmax()))
        ref.append(seq[len(p):])
    llm = LLM(model, dtype="float32", max_model_len=64, max_num_seqs=2, max_batched_tokens=64, pass_tokens=64, block_size=16,
              kv_blocks=8, policy="chunked", chunk=8, eager=eager, capture_at_start=False)
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=new, ignore_eos=True))
    assert [o["token_ids"] for o in outs] == ref
    assert llm.executor.cache.all_free()
    if not eager:
        assert llm.executor.n_graph_steps > 0


def test_a_model_folder_through_the_replay_program_and_the_command_line(tmp_path):
    """A Sarulix folder written by the random-weights mode, with the low ranks left to the tensors' shapes:
    `bin/trace_run` replays a trace of five requests on four state slots and a pool smaller than their sum (float32
    logits against the plain model), and `python -m llmgen_b200 chat` generates the plain model's greedy tokens."""
    import json
    import os
    import subprocess
    import sys

    import numpy as np
    from safetensors.torch import load_file

    from llmgen_b200.engine.api import write_random_model
    from tests.util import ROOT
    cfg = su.MIXED
    folder = write_random_model(str(tmp_path / "model"), cfg, seed=12, sigma=0.1, sigma_norm=0.2)
    path = os.path.join(folder, "config.json")
    with open(path) as f:
        written = json.load(f)
    assert written["architecture"] == "Sarulix"
    for key in ("decay_rank", "gate_rank"):       # as a folder from elsewhere has it: the shapes say it
        del written["layers"][1]["mixer"][key]
    with open(path, "w") as f:
        json.dump(written, f)
    tensors = load_file(os.path.join(folder, "model.safetensors"))
    lengths = [70, 40, 23, 64, 51]
    ids = [su.ids_for(cfg, n, 70 + i) for i, n in enumerate(lengths)]
    want = [su.plain_logits(cfg, tensors, t) for t in ids]
    steps, pos, live, waiting = [], [0] * 5, [0, 1, 2, 3], [4]
    portions = [17, 2, 1, 30, 1, 1, 64]
    k = 0
    while live:
        entries, ended = [], []
        for r in live:
            n = min(portions[(k + r) % len(portions)], lengths[r] - pos[r])
            entries.append((r, pos[r], pos[r] + n))
            pos[r] += n
            if pos[r] == lengths[r]:
                ended.append(r)
        steps.append((entries, ended))
        live = [r for r in live if r not in ended]
        if ended and waiting:
            live.append(waiting.pop(0))
        k += 1
    lines = [json.dumps({"step": i, "entries": [{"id": f"r{r}", "tokens": ids[r][lo:hi], "want": list(range(hi - lo))} for r, lo, hi in entries],
                         "end": [f"r{r}" for r in ended]}) for i, (entries, ended) in enumerate(steps)]
    out_dir = str(tmp_path / "out")
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", "float32", "--out", out_dir,
                           "--max-tokens", "256"], input="\n".join(lines) + "\n", capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(len(steps))]
    for i, (entries, _) in enumerate(steps):
        got = torch.from_numpy(np.fromfile(os.path.join(out_dir, f"{i}.f32"), dtype="<f4").reshape(-1, cfg["vocab"]))
        ref = torch.cat([want[r][lo:hi] for r, lo, hi in entries])
        assert su.relative_error(got, ref) < su.TOL["float32"], i
    prompt, new = ids[2][:9], 8
    seq = list(prompt)
    for _ in range(new):
        seq.append(int(su.plain_logits(cfg, tensors, seq)[-1].argmax()))
    proc = subprocess.run([sys.executable, "-m", "llmgen_b200", "chat", ",".join(map(str, prompt)), str(new), "--model", folder, "--dtype", "float32",
                           "--max-model-len", "64", "--max-num-seqs", "2", "--max-batched-tokens", "64", "--kv-blocks", "8"],
                          capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert proc.returncode == 0, proc.stderr[-2000:]
    printed = [l.split() for l in proc.stdout.splitlines() if l.split() and all(t.lstrip("-").isdigit() for t in l.split())]
    assert printed and [int(t) for t in printed[-1]] == seq[len(prompt):], proc.stdout[-2000:]
