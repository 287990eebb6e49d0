"""Tafesun through the engine against the plain implementation (GPU): every way of cutting the
work, tiny configurations that differ in every size and option, float32 and bfloat16."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import gpu_harness as H
import tafesun_configs as C
from plain import tafesun_plain as P

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
F32_FRAC = 2e-5
LENGTHS = (1, 2, 9, 40, 77, 131, 203)


def refs_of(cfg, weights, seqs):
    return [P.forward(cfg, weights, s, torch.float64) for s in seqs]


class Case:
    """A configuration with two sets of weights: freely routed tokens for float32, decisive routers for bfloat16
    (see tafesun_configs.decisive_routers)."""

    def __init__(self, which, tmp, lengths=LENGTHS, seq_seed=7, seed=None, edit=None):
        self.which = which
        seed = ord(which[0]) if seed is None else seed
        self.by_dtype = {}
        for dtype, routers in (("float32", None), ("bfloat16", C.decisive_routers)):
            def both(w, routers=routers):
                if edit:
                    edit(w)
                if routers:
                    routers(w)
            d, cfg, weights = C.make_model_dir(which, str(tmp / dtype), seed=seed, edit=both)
            self.cfg = cfg
            self.seqs = C.sequences(cfg, lengths, seed=seq_seed)
            self.by_dtype[dtype] = (d, weights, refs_of(cfg, weights, self.seqs))

    def of(self, dtype):
        return self.by_dtype[dtype]


@pytest.fixture(scope="module", params=["A", "B", "C"])
def case(request, tmp_path_factory):
    return Case(request.param, tmp_path_factory.mktemp(f"tf{request.param}"))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("cutting", ["whole", "tail", "portions", "mixed"])
def test_cuttings_agree_with_plain(case, dtype, cutting):
    which, seqs = case.which, case.seqs
    d, weights, refs = case.of(dtype)
    page_size = 16
    if cutting == "mixed":
        # so few pages and slots that they are used again
        budget = max((len(s) + page_size - 1) // page_size for s in seqs) + 5
        runner = H.make_runner(d, dtype, page_size=page_size, num_pages=budget, num_slots=3)
        script = H.script_mixed(seqs, max_live=3, seed=5, budget_pages=budget, page_size=page_size)
        assert any(len(p) > 1 and any(n == 1 for _, _, n in p) and any(n > 1 for _, _, n in p) for p, _ in script)
    else:
        runner = H.make_runner(d, dtype, page_size=page_size, num_pages=16, num_slots=2)
        script = {"whole": H.script_whole, "portions": H.script_portions,
                  "tail": lambda s: H.script_tail_one_by_one(s, tail=70)}[cutting](seqs)
    out = H.run_script(runner, seqs, script)
    for i, ref in enumerate(refs):
        H.check_rows(out[i], ref, dtype, f"{which} {dtype} {cutting} seq {i} (len {len(seqs[i])})", f32_frac=F32_FRAC)
    for g in runner.cache.groups.values():
        assert g.pool.n_free == g.num_pages  # every page came back
    assert runner.cache.free_slots == runner.cache.num_slots


@pytest.mark.parametrize("page_size", [16, 64])
def test_portions_of_two_tokens_and_page_borders(case, page_size):
    """Every portion is two tokens long (then three, so that both parities of a page's edge are met),
    against the whole prompt."""
    which, seqs = case.which, case.seqs
    d, weights, refs = case.of("float32")
    i = 5
    for width in (2, 3):
        runner = H.make_runner(d, "float32", page_size=page_size, num_pages=max(4, 256 // page_size), num_slots=1)
        n = len(seqs[i])
        script = [([(i, a, min(width, n - a))], [i] if a + width >= n else []) for a in range(0, n, width)]
        out = H.run_script(runner, seqs, script)
        H.check_rows(out[i], refs[i], "float32", f"{which} portions of {width}", f32_frac=F32_FRAC)


def test_long_decoding_from_the_first_token(case):
    """One prompt token, then 202 tokens one by one: the state and the convolution's last inputs are
    carried 200 steps, the keys of decoded tokens fill page after page."""
    which, seqs = case.which, case.seqs
    for dtype in ("float32", "bfloat16"):
        d, weights, refs = case.of(dtype)
        runner = H.make_runner(d, dtype, page_size=16, num_pages=16, num_slots=1)
        out = H.run_script(runner, seqs[6:7], H.script_tail_one_by_one(seqs[6:7], tail=len(seqs[6]) - 1))
        H.check_rows(out[0], refs[6], dtype, f"{which} {dtype} long decoding", f32_frac=F32_FRAC)


def test_batch_of_unequal_requests_equals_each_alone(case):
    which, seqs = case.which, case.seqs
    for dtype in ("float32", "bfloat16"):
        d, weights, refs = case.of(dtype)
        runner = H.make_runner(d, dtype, page_size=16, num_pages=40, num_slots=4)
        pick = [1, 3, 4, 6]
        half = {i: len(seqs[i]) // 2 for i in pick}
        script = [([(i, 0, half[i]) for i in pick], []),
                  ([(i, half[i], len(seqs[i]) - half[i]) for i in pick], pick)]
        out = H.run_script(runner, seqs, script)
        for i in pick:
            H.check_rows(out[i], refs[i], dtype, f"{which} {dtype} batched seq {i}", f32_frac=F32_FRAC)


def test_slot_and_pages_used_again_start_clean(case):
    """A request that takes the slot and pages of a finished one sees nothing of it."""
    which, seqs = case.which, case.seqs
    d, weights, refs = case.of("float32")
    runner = H.make_runner(d, "float32", page_size=16, num_pages=13, num_slots=1)
    script = [([(6, 0, 203)], [6]), ([(5, 0, 50)], []), ([(5, 50, 81)], [5]), ([(3, 0, 40)], [3])]
    out = H.run_script(runner, seqs, script)
    for i in (6, 5, 3):
        H.check_rows(out[i], refs[i], "float32", f"{which} reuse seq {i}", f32_frac=F32_FRAC)


def _loud_far_key(weights, cfg):
    """Layer 0's first query head asks for one key far back: its query and key projections are made
    large along one unrotated channel pair, so that a single score stands out by far."""
    L = cfg["layers"][0]["mixer"]["left"]
    d = L["dim"]
    ch = d - 1  # the last channel of the head is outside the rotated part in configuration A
    for name in ("l0.mix.left.q", "l0.mix.left.k"):
        w = weights[name]
        w[ch] = w[ch] * 12.0


def test_loud_far_key_and_slow_state(tmp_path):
    """Weights under which a lost key, a lost state or a gate left out cannot hide: one attention head
    puts nearly all its weight on single keys wherever they lie (hundreds of tokens back, across
    pages), and the state-space heads barely forget (their step sizes are small), so that the first
    tokens weigh in the last ones' outputs."""
    def edit(w):
        _loud_far_key(w, C.TF_A)
        w["l0.mix.right.dt_bias"] = w["l0.mix.right.dt_bias"] - 3.0
        w["l0.mix.right.A_log"] = w["l0.mix.right.A_log"] - 2.0
    case = Case("A", tmp_path, lengths=(300,), seq_seed=3, seed=11, edit=edit)
    seqs, cfg = case.seqs, case.cfg
    for dtype in ("float32", "bfloat16"):
        d, weights, refs = case.of(dtype)
        ref = refs[0]
        # the oracle itself: with the far tokens changed the last logits move visibly
        other = list(seqs[0])
        other[:40] = C.sequences(cfg, (40,), seed=99)[0]
        assert float((P.forward(cfg, weights, other, torch.float64)[-20:] - ref[-20:]).abs().max()) > 0.05
        for script in (H.script_whole(seqs), H.script_tail_one_by_one(seqs, tail=64), H.script_portions(seqs, seed=2)):
            runner = H.make_runner(d, dtype, page_size=16, num_pages=24, num_slots=1)
            out = H.run_script(runner, seqs, script)
            H.check_rows(out[0], ref, dtype, f"loud {dtype}", f32_frac=4e-5)


def test_greedy_generation_through_the_engine(case):
    """Engine.generate (scheduler, sampler, decode graphs) against greedy decoding with the plain
    implementation, float32; bfloat16 with graphs against bfloat16 step by step."""
    from poor_mans_mamba_b200.entry import Engine
    which, seqs, cfg = case.which, case.seqs, case.cfg
    d, weights, refs = case.of("float32")
    prompts = [seqs[2], seqs[3][:23], seqs[1]]
    n_new = 12
    eng = Engine(d, dtype="float32", max_tokens=1024, max_seqs=4, page_size=16, max_batched_tokens=32)
    got = eng.generate(prompts, max_new_tokens=n_new, eos_token_id=-1)
    for p, g in zip(prompts, got):
        toks = list(p)
        for _ in range(n_new):
            lg = P.forward(cfg, weights, toks, torch.float64)[-1]
            top2 = torch.topk(lg, 2).values
            if float(top2[0] - top2[1]) < 1e-3:
                break  # a near tie: the two may disagree from here on without either being wrong
            toks.append(int(lg.argmax()))
        want = toks[len(p):]
        assert g[:len(want)] == want
    d = case.of("bfloat16")[0]
    a = Engine(d, dtype="bfloat16", max_tokens=1024, max_seqs=4, page_size=16, cuda_graphs=True).generate(
        prompts, max_new_tokens=n_new, eos_token_id=-1)
    b = Engine(d, dtype="bfloat16", max_tokens=1024, max_seqs=4, page_size=16, cuda_graphs=False).generate(
        prompts, max_new_tokens=n_new, eos_token_id=-1)
    assert a == b


def test_trace_program_replays_a_schedule(case, tmp_path):
    which, seqs, cfg = case.which, case.seqs, case.cfg
    if which != "A":
        pytest.skip("one configuration is enough for the program")
    steps = [
        {"step": 0, "entries": [{"id": "x", "tokens": seqs[3][:17], "want": [0, 16]},
                                {"id": "y", "tokens": seqs[2], "want": [8]}], "end": ["y"]},
        {"step": 1, "entries": [{"id": "x", "tokens": seqs[3][17:19], "want": []}], "end": []},
        {"step": 2, "entries": [{"id": "x", "tokens": seqs[3][19:], "want": [len(seqs[3]) - 20]},
                                {"id": "z", "tokens": seqs[1], "want": [1]}], "end": ["x", "z"]},
    ]
    for dtype in ("float32", "bfloat16"):
        d, weights, refs = case.of(dtype)
        out_dir = str(tmp_path / f"out_{dtype}")
        proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", d, "--dtype", dtype,
                               "--out", out_dir, "--max-tokens", "128"],
                              input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True,
                              timeout=600)
        assert proc.returncode == 0, proc.stderr[-2000:]
        assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
        V = cfg["vocab"]
        s0 = np.fromfile(os.path.join(out_dir, "0.f32"), dtype="<f4").reshape(-1, V)
        s2 = np.fromfile(os.path.join(out_dir, "2.f32"), dtype="<f4").reshape(-1, V)
        assert not os.path.exists(os.path.join(out_dir, "1.f32"))
        want0 = torch.stack([refs[3][0], refs[3][16], refs[2][8]])
        want2 = torch.stack([refs[3][-1], refs[1][1]])
        H.check_rows(torch.from_numpy(s0), want0, dtype, "trace step 0", f32_frac=F32_FRAC)
        H.check_rows(torch.from_numpy(s2), want2, dtype, "trace step 2", f32_frac=F32_FRAC)


def test_command_line_generates_from_a_model_folder(case):
    which, seqs, cfg = case.which, case.seqs, case.cfg
    d, weights, refs = case.of("float32")
    if which != "B":
        pytest.skip("one configuration is enough for the program")
    prompt = ",".join(str(t) for t in seqs[2])
    proc = subprocess.run([sys.executable, "-m", "poor_mans_mamba_b200", d, "64", "GPU", "1", "2", "5", "--dtype", "float32",
                           "--prompt-ids", prompt, "--page-size", "16"], capture_output=True, text=True, timeout=600,
                          cwd=ROOT)
    assert proc.returncode == 0, proc.stderr[-2000:]
    lines = [l for l in proc.stdout.splitlines() if l.startswith("req_id=")]
    assert len(lines) == 2 and all("gen_tokens=5" in l for l in lines)
    toks = list(seqs[2])
    for _ in range(5):
        toks.append(int(P.forward(cfg, weights, toks, torch.float64)[-1].argmax()))
    assert str(toks[len(seqs[2]):]) in lines[0]


def test_medium_sizes_where_the_tensor_core_forms_run(tmp_path):
    """Head sizes of 64 and 128, a padded value size, prompts long enough for the tcgen05 attention and the
    chunked scan, expert rows that the tensor-core grouped products take, pages of 64 tokens: whole, in
    portions that cut chunks anywhere, and with a long tail decoded through the decode attention."""
    case = Case("M", tmp_path, lengths=(700, 333), seq_seed=9, seed=21)
    seqs = case.seqs
    for dtype in ("float32", "bfloat16"):
        d, weights, refs = case.of(dtype)
        for name, script in (("whole", H.script_whole(seqs)),
                             ("tail", H.script_tail_one_by_one(seqs, tail=80)),
                             ("portions", [([(0, 0, 257)], []), ([(0, 257, 2), (1, 0, 130)], []),
                                           ([(0, 259, 300), (1, 130, 1)], []), ([(0, 559, 141), (1, 131, 202)], [0, 1])])):
            runner = H.make_runner(d, dtype, page_size=64, num_pages=20, num_slots=2)
            out = H.run_script(runner, seqs, script)
            for i, ref in enumerate(refs):
                H.check_rows(out[i], ref, dtype, f"medium {dtype} {name} seq {i}", f32_frac=4e-5)
