"""CPU: the host side of the Lugovik family: configuration reader, safetensors reader, weight stacking, rotation
frequencies, the ABI of libb200seq, and the engine's scheduler and slot bookkeeping over a stand-in model."""
import ctypes as C
import json
import os
import re
import subprocess

import pytest
import torch

import lugovik_oracle as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_seq_abi_matches_the_header(tmp_path):
    from lit_llama_b200 import _seqlib as S

    src = re.sub(r"/\*.*?\*/", "", open(os.path.join(ROOT, "include", "b2l_seq.h")).read(), flags=re.S)
    names = sorted(set(re.findall(r"\b(b2l_seq_[a-z0-9_]+)\s*\(", src)))
    assert sorted(S.EXPORTS) == names
    handle = C.CDLL(S._build.ensure("seq"))
    for n in names:
        assert hasattr(handle, n), n
    prog = tmp_path / "layout.c"
    prog.write_text('#include <stdio.h>\n#include <stddef.h>\n#include "b2l_seq.h"\nint main(void){printf("%zu %zu %zu %zu %zu %zu\\n", '
                    "sizeof(b2l_seq_scan_args), sizeof(b2l_seq_attn_args), offsetof(b2l_seq_scan_args, decay), offsetof(b2l_seq_scan_args, act_dtype), "
                    "offsetof(b2l_seq_attn_args, scale), offsetof(b2l_seq_attn_args, act_dtype));return 0;}\n")
    exe = tmp_path / "layout"
    subprocess.run(["gcc", "-I", os.path.join(ROOT, "include"), str(prog), "-o", str(exe)], check=True)
    out = [int(v) for v in subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split()]
    assert out == [C.sizeof(S.ScanArgs), C.sizeof(S.AttnArgs), S.ScanArgs.decay.offset, S.ScanArgs.act_dtype.offset, S.AttnArgs.scale.offset,
                   S.AttnArgs.act_dtype.offset]
    assert S.lib().b2l_seq_version() == 100


def test_safetensors_round_trip(tmp_path):
    from lit_llama_b200.checkpoint_io import read_safetensors, write_safetensors

    t = {"a.b": torch.randn(3, 5).bfloat16(), "n": torch.arange(7, dtype=torch.int32), "f": torch.randn(2, 2, 2), "empty": torch.zeros(0, 4)}
    path = str(tmp_path / "m.safetensors")
    write_safetensors(path, t)
    back = read_safetensors(path)
    assert set(back) == set(t) and all(torch.equal(back[k], t[k]) and back[k].dtype == t[k].dtype for k in t)
    conv = read_safetensors(path, float_dtype=torch.float32)
    assert conv["a.b"].dtype == torch.float32 and conv["n"].dtype == torch.int32
    with open(path, "r+b") as f:      # a tensor that does not fit its shape is refused
        f.seek(8)
        head = f.read(200)
        f.seek(8)
        f.write(head.replace(b'"shape":[3,5]', b'"shape":[3,6]'))
    with pytest.raises(ValueError):
        read_safetensors(path)


def test_configuration_reader():
    from lit_llama_b200.lugovik import LugovikConfig

    d = {"architecture": "Lugovik", "vocab": 9, "width": 4, "norm": {"eps": 1e-5}, "layers": [
        {"type": "mamba2", "mlp": None, "mixer": {"conv": 2, "heads": 1, "state": 4, "vdim": 4}}]}
    c = LugovikConfig.from_dict(d)
    assert (c.vocab, c.width, c.eps, c.embedding_scale) == (9, 4, 1e-5, 1.0) and c.to_dict()["layers"] == d["layers"]
    for bad in ({**d, "architecture": "Other"}, {**d, "layers": [{"type": "x"}]},
                {**d, "layers": [{"type": "mamba2", "mlp": {"kind": "sparse"}, "mixer": {}}]}):
        with pytest.raises(ValueError):
            LugovikConfig.from_dict(bad)


def test_registry_knows_both_families(tmp_path):
    from lit_llama_b200 import registry

    assert {"LLaMA", "Lugovik"} <= set(registry.architectures())
    (tmp_path / "config.json").write_text(json.dumps({"architecture": "Nobody"}))
    with pytest.raises(ValueError):
        registry.load_model(str(tmp_path), device="cpu")


def test_weight_stacking_and_frequencies():
    from lit_llama_b200.mixers import rope_frequencies, stack_rows

    a, b, c = torch.randn(5, 3), torch.randn(8, 3), torch.randn(1, 3)
    w, offs = stack_rows([a, b, c])
    assert offs == [0, 8, 16] and w.shape == (24, 3)
    assert torch.equal(w[0:5], a) and torch.equal(w[8:16], b) and torch.equal(w[16:17], c) and float(w[5:8].abs().sum() + w[17:].abs().sum()) == 0
    for rot in ({"base": 1e4, "dims": 64}, {"base": 5e5, "dims": 32, "scaling": {"factor": 16.0, "original": 2048, "fast": 32.0, "slow": 1.0}},
                {"base": 100.0, "dims": 8, "scaling": {"factor": 2.0, "original": 8, "fast": 1.0, "slow": 1.0}}):
        f, m = rope_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
        fo, mo = O.rope_frequencies(rot)
        assert torch.allclose(f.double(), fo, rtol=1e-7, atol=0) and abs(m - mo) < 1e-12


def test_oracle_whole_equals_its_own_prefix():
    """The plain model is causal: logits of a prefix do not change when tokens follow."""
    cfg = {"architecture": "Lugovik", "vocab": 31, "width": 16, "norm": {"eps": 1e-6}, "embedding": {"scale": 2.0}, "layers": [
        {"type": "channel_delta", "mlp": {"kind": "dense", "ff": 24}, "mixer": {"conv": 3, "dim": 4, "heads": 2, "kv_heads": 1, "vdim": 6}},
        {"type": "parallel", "mlp": None, "mixer": {"left": {"heads": 2, "kv_heads": 1, "dim": 8, "vdim": 4, "mask": {"size": 3}, "scale": 0.3,
                                                               "softcap": 10.0, "rot": {"base": 100.0, "dims": 4}},
                                                      "right": {"heads": 1, "dim": 4, "vdim": 4, "tau": 2.0}, "left_scale": 1.0, "right_scale": 0.5}},
        {"type": "mamba2", "mlp": None, "mixer": {"conv": 2, "groups": 1, "heads": 2, "norm_groups": 2, "state": 4, "vdim": 4}}]}
    W = {k: v.double() for k, v in O.random_weights(cfg, seed=2).items()}
    toks = [1, 5, 30, 2, 2, 17, 9, 0, 4]
    full = O.forward(cfg, W, toks)
    assert torch.allclose(O.forward(cfg, W, toks[:6]), full[:6], rtol=1e-10, atol=1e-12)
    assert full.shape == (9, 31) and bool(torch.isfinite(full).all())


class _CountingModel:
    """Stand-in for the scheduler tests: no state, logits point at (sum of the sequence's tokens so far) % vocab."""
    graph_safe = False
    vocab, dtype, device = 13, torch.float32, torch.device("cpu")

    def __init__(self):
        self.calls, self.sums = [], {}

    def state_specs(self):
        return {}

    def forward_portion(self, tokens, ctx, want=None):
        slot, pos0 = int(ctx.meta[0]), int(ctx.meta[1])
        if pos0 == 0:
            self.sums[slot] = 0
        self.calls.append((slot, pos0, tokens.numel()))
        out = []
        for t in tokens.tolist():
            self.sums[slot] += t
            row = torch.zeros(self.vocab)
            row[self.sums[slot] % self.vocab] = 1.0
            out.append(row)
        out = torch.stack(out)
        return out if want is None else out[want.long()]


def test_scheduler_portions_turns_slots_and_budget():
    from lit_llama_b200.engine import Engine
    from lit_llama_b200.state import PoolFull

    def expect(prompt, n):
        seq = list(prompt)
        for _ in range(n):
            seq.append(sum(seq) % 13)
        return seq[len(prompt):]

    m = _CountingModel()
    e = Engine(m, n_slots=2, prefill_chunk=4, device="cpu")
    prompts = {"a": [1, 2, 3, 4, 5, 6, 7, 8, 9], "b": [5], "c": [3, 3, 3, 3, 3], "d": [12, 1]}
    for k, p in prompts.items():
        e.add_request(k, p, 5)
    with pytest.raises(KeyError):
        e.add_request("a", [1], 1)
    out = e.run()
    assert out == {k: expect(p, 5) for k, p in prompts.items()}
    assert max(c[2] for c in m.calls) <= 4 and e.pool.free_slots() == 2 and e.pool.reused >= 2
    assert [c[2] for c in m.calls if c[0] == 0][:3] == [4, 4, 1]          # request a: portions of the prompt, in order
    # eos ends a request early, and the token is kept
    e.add_request("e", [1, 1], 10, eos_id=expect([1, 1], 3)[2])
    assert e.run()["e"] == expect([1, 1], 3)
    # caller-scheduled steps keep positions per request and give slots back at `end`
    e.step([{"id": "p", "tokens": [1, 2], "want": []}, {"id": "q", "tokens": [4], "want": [0]}])
    assert e.pool.position("p") == 2 and e.pool.position("q") == 1 and e.pool.free_slots() == 0
    with pytest.raises(PoolFull):
        e.step([{"id": "r", "tokens": [1], "want": []}])
    got = e.step([{"id": "p", "tokens": [3], "want": [0]}], end=["p", "q"])[0]
    assert int(got.argmax()) == 6 and e.pool.free_slots() == 2
    with pytest.raises(IndexError):
        e.step([{"id": "s", "tokens": [1], "want": [1]}], end=["s"])
    # a token budget keeps requests waiting instead of overbooking
    e2 = Engine(_CountingModel(), n_slots=4, max_tokens=12, device="cpu")
    for i in range(3):
        e2.add_request(i, [1, 2, 3], 3)
    assert e2.run() == {i: expect([1, 2, 3], 3) for i in range(3)}
    e2.add_request("big", [1] * 20, 1)
    with pytest.raises(PoolFull):
        e2.run()
