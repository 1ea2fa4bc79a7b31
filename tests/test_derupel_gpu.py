"""Derupel through the engine against the plain implementation (tests/plain/derupel_plain.py, float64 on the CPU):
whole prompts, portions, token by token, batches, pages and state slots used again, graphs replayed, generation."""
import pytest
import torch

from tests import derupel_util as du

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["MIXED", "WIDE", "ODD"])
def test_whole_prompt_and_portions_match_the_plain_model(name, dtype):
    cfg = getattr(du, name)
    model, tensors = du.build(cfg, seed=3, dtype=dtype)
    ids = du.ids_for(cfg, 75, seed=1)
    want = du.plain_logits(cfg, tensors, ids)
    drv = du.driver(model, dtype)
    du.assert_close(du.run_in_portions(drv, "a", ids, [len(ids)]), want, dtype)
    du.assert_close(du.run_in_portions(drv, "a", ids, [33, 2, 1, 17, 1]), want, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_portions_of_any_size_and_single_tokens_give_the_whole_prompts_logits(dtype):
    cfg = du.MIXED
    model, tensors = du.build(cfg, seed=4, dtype=dtype)
    ids = du.ids_for(cfg, 101, seed=2)
    want = du.plain_logits(cfg, tensors, ids)
    drv = du.driver(model, dtype)
    for portions in ([1], [2], [3, 2, 33, 31, 1, 16, 2], [32, 32, 5, 1], [47, 1, 1, 2]):
        got = du.run_in_portions(drv, "a", ids, portions)
        du.assert_close(got, want, dtype, portions)
    assert drv.executor.cache.all_free()


@pytest.mark.parametrize("eager", [True, False])
@pytest.mark.parametrize("dtype", DTYPES)
def test_unequal_requests_in_one_batch_match_each_alone(dtype, eager):
    """Three requests of different lengths, portions of some beside single tokens of others; launched kernel by kernel and
    replayed from the graphs of the steps' shapes."""
    cfg = du.MIXED
    model, tensors = du.build(cfg, seed=5, dtype=dtype)
    ids = {"a": du.ids_for(cfg, 70, 11), "b": du.ids_for(cfg, 19, 12), "c": du.ids_for(cfg, 41, 13)}
    want = {r: du.plain_logits(cfg, tensors, t) for r, t in ids.items()}
    drv = du.driver(model, dtype, eager=eager)
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
        du.assert_close(torch.cat(got[r]), want[r], dtype, r)
    if not eager:
        assert drv.executor.n_shaped_steps > 0


@pytest.mark.parametrize("dtype", DTYPES)
def test_pages_and_state_slots_are_used_again(dtype):
    """A pool of 6 pages and 2 state slots, five requests one after and beside another: every page and slot serves
    several requests, and a request that starts in a used slot starts from an empty state."""
    cfg = du.MIXED
    model, tensors = du.build(cfg, seed=6, dtype=dtype)
    drv = du.driver(model, dtype, pool_tokens=96, page_size=16, max_num_seqs=2)
    lengths = [40, 50, 33, 17, 48]
    all_ids = [du.ids_for(cfg, n, 20 + i) for i, n in enumerate(lengths)]
    want = [du.plain_logits(cfg, tensors, t) for t in all_ids]
    slots_seen = set()
    # 0 alone, then 1 with 2 (1 in portions, 2 token by token after its first 20), then 3 with 4
    got0 = du.run_in_portions(drv, 0, all_ids[0], [13, 27])
    du.assert_close(got0, want[0], dtype)
    for pair in ((1, 2), (3, 4)):
        a, b = pair
        ga, gb = [], []
        pa = pb = 0
        while pa < lengths[a] or pb < lengths[b]:
            entries, end = [], []
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
        du.assert_close(torch.cat(ga), want[a], dtype, a)
        du.assert_close(torch.cat(gb), want[b], dtype, b)
    assert slots_seen == {0, 1}
    assert drv.executor.cache.all_free()


@pytest.mark.parametrize("needle_at", [0, 3, 15, 16, 17, 255, 256, 298])
def test_one_key_decides_wherever_it_lies(needle_at):
    """The last token's query finds the key of one token only (`plant_needle`): far back, the first of the sequence, on
    either side of a page's border (pages of 16), the newest but one; in a whole prompt, in portions cut at and beside
    the needle, and with the probe decoded alone after single tokens.  Without the needle the oracle's own last row
    moves by thousands of tolerances, so a key or value taken from the wrong place could not hide."""
    cfg = du.NEEDLE
    model, tensors = du.build(cfg, seed=7, dtype="float32", sigma=0.3, prepare=du.plant_needle)
    n = 300
    ids = du.needle_ids(cfg, n, needle_at, 31)
    want = du.plain_logits(cfg, tensors, ids)
    without = list(ids)
    without[needle_at] = du.FILLER_ID
    assert du.relative_error(du.plain_logits(cfg, tensors, without)[-1:], want[-1:]) > 1000 * du.TOL["float32"]
    drv = du.driver(model, "float32", pool_tokens=320)
    cut = max(needle_at, 1)
    for portions in ([n], [cut, 1, 2, n], [needle_at + 1, 1, n], [290] + [1] * 10):
        got = du.run_in_portions(drv, "a", ids, portions)
        assert du.relative_error(got, want) < du.TOL["float32"], portions


def test_a_state_that_forgets_nothing_is_carried_through_portions_and_long_decoding():
    cfg = du.KEEPING
    model, tensors = du.build(cfg, seed=8, dtype="float32")
    ids = du.ids_for(cfg, 400, 41)
    want = du.plain_logits(cfg, tensors, ids)
    drv = du.driver(model, "float32", pool_tokens=448)
    for portions in ([400], [31, 33, 32, 1, 2, 64, 1], [100] + [1] * 300):
        got = du.run_in_portions(drv, "a", ids, portions)
        assert du.relative_error(got, want) < du.TOL["float32"], portions[:3]
    # the first token still counts at the end: without it the last logits differ
    shifted = du.plain_logits(cfg, tensors, ids[1:])
    assert du.relative_error(shifted[-1:], want[-1:]) > 100 * du.TOL["float32"]


def test_the_first_tokens_of_a_sequence():
    cfg = du.MIXED
    model, tensors = du.build(cfg, seed=9, dtype="float32")
    drv = du.driver(model, "float32")
    for n in (1, 2, 3):
        ids = du.ids_for(cfg, n, 50 + n)
        got = du.run_in_portions(drv, "a", ids, [1])
        assert du.relative_error(got, du.plain_logits(cfg, tensors, ids)) < du.TOL["float32"]


@pytest.mark.parametrize("eager", [True, False])
def test_greedy_generation_through_the_engine_and_its_scheduler(eager):
    """`LLM.generate` (scheduler, chunked prompts, decode graphs, sampling kernel) against greedy decoding with the
    plain model."""
    from llmgen_b200.engine.api import LLM
    from llmgen_b200.sampling.params import SamplingParams
    cfg = du.MIXED
    model, tensors = du.build(cfg, seed=10, dtype="float32")
    prompts = [du.ids_for(cfg, n, 60 + n) for n in (9, 21, 4)]
    new = 10
    ref = []
    for p in prompts:
        seq = list(p)
        for _ in range(new):
            seq.append(int(du.plain_logits(cfg, tensors, seq)[-1].argmax()))
        ref.append(seq[len(p):])
    llm = LLM(model, dtype="float32", max_model_len=64, max_num_seqs=2, max_batched_tokens=64, pass_tokens=64, block_size=16,
              kv_blocks=8, policy="chunked", chunk=8, eager=eager, capture_at_start=False)
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=new, ignore_eos=True))
    assert [o["token_ids"] for o in outs] == ref
    assert llm.executor.cache.all_free()
    if not eager:
        assert llm.executor.n_graph_steps > 0


def test_a_model_folder_through_the_replay_program_and_the_command_line(tmp_path):
    """A Derupel folder written by the random-weights mode: `bin/trace_run` replays a trace of five requests on four state
    slots and a pool smaller than their sum (float32 logits against the plain model), and `python -m llmgen_b200 chat`
    generates the plain model's greedy tokens."""
    import json
    import os
    import subprocess
    import sys

    import numpy as np
    from safetensors.torch import load_file

    from llmgen_b200.engine.api import write_random_model
    from tests.util import ROOT
    cfg = du.MIXED
    folder = write_random_model(str(tmp_path / "model"), cfg, seed=12, sigma=0.1, sigma_norm=0.2)
    with open(os.path.join(folder, "config.json")) as f:
        assert json.load(f)["architecture"] == "Derupel"
    tensors = load_file(os.path.join(folder, "model.safetensors"))
    lengths = [70, 40, 23, 64, 51]
    ids = [du.ids_for(cfg, n, 70 + i) for i, n in enumerate(lengths)]
    want = [du.plain_logits(cfg, tensors, t) for t in ids]
    # requests 0-3 in portions side by side; 4 comes when 2 has ended and takes its slot and pages
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
        assert du.relative_error(got, ref) < du.TOL["float32"], i
    # the command line: greedy generation from a prompt of token ids
    prompt, new = ids[2][:9], 8
    seq = list(prompt)
    for _ in range(new):
        seq.append(int(du.plain_logits(cfg, tensors, seq)[-1].argmax()))
    proc = subprocess.run([sys.executable, "-m", "llmgen_b200", "chat", ",".join(map(str, prompt)), str(new), "--model", folder, "--dtype", "float32",
                           "--max-model-len", "64", "--max-num-seqs", "2", "--max-batched-tokens", "64", "--kv-blocks", "8"],
                          capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert proc.returncode == 0, proc.stderr[-2000:]
    printed = [l.split() for l in proc.stdout.splitlines() if l.split() and all(t.lstrip("-").isdigit() for t in l.split())]
    assert printed and [int(t) for t in printed[-1]] == seq[len(prompt):], proc.stdout[-2000:]
