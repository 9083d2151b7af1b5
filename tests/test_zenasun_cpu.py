"""CPU: the host side of the Zenasun family: configuration reader, registry entry, the argument block of the latent
attention against a C compiler, and the plain restatement against itself (whole sequence = carried state)."""
import ctypes as C
import os
import subprocess

import pytest
import torch

import zenasun_oracle as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _cfg():
    la = {"heads": 2, "dim": 4, "rot_dim": 2, "vdim": 6, "q_rank": 5, "kv_rank": 3, "scale": 0.5, "rot": {"base": 10.0, "dims": 2}}
    return {"architecture": "Zenasun", "vocab": 9, "width": 8, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.0}, "layers": [
        {"type": "latent_attention", "mixer": la, "mlp": None},
        {"type": "retention", "mixer": {"heads": 1, "dim": 4, "vdim": 2, "decay": [0.5], "rot": {"base": 10.0, "dims": 2}},
         "mlp": {"kind": "moe", "expert": {"ff": 4}, "router": {"experts": 2, "identity": 1, "top": 1, "groups": {"count": 1, "keep": 1}}}},
        {"type": "latent_attention", "mixer": la, "mlp": None, "weights_of": 0}]}


def test_configuration_reader():
    from lit_llama_b200.zenasun import ZenasunConfig

    d = _cfg()
    c = ZenasunConfig.from_dict(d)
    assert (c.vocab, c.width, c.eps, c.embedding_scale, c.logit_softcap) == (9, 8, 1e-5, 2.0, None)
    assert ZenasunConfig.from_dict({**d, "logit_softcap": 25}).logit_softcap == 25.0
    assert c.to_dict()["layers"] == d["layers"]
    bad_share = [dict(x) for x in d["layers"]]
    bad_share[2]["weights_of"] = 1            # a layer of another type
    bad_kind = [dict(x) for x in d["layers"]]
    bad_kind[1] = {**bad_kind[1], "mlp": {"kind": "dense"}}
    for bad in ({**d, "architecture": "Other"}, {**d, "layers": [{"type": "x"}]}, {**d, "layers": bad_share}, {**d, "layers": bad_kind}):
        with pytest.raises(ValueError):
            ZenasunConfig.from_dict(bad)


def test_registry_knows_the_family():
    from lit_llama_b200 import registry

    assert {"LLaMA", "Lugovik", "Zenasun"} <= set(registry.architectures())


def test_latent_argument_block_matches_the_header(tmp_path):
    from lit_llama_b200 import _seqlib as S

    prog = tmp_path / "layout.c"
    prog.write_text('#include <stdio.h>\n#include <stddef.h>\n#include "b2l_seq.h"\nint main(void){printf("%zu %zu %zu %zu %zu\\n", '
                    "sizeof(b2l_seq_latent_attn_args), offsetof(b2l_seq_latent_attn_args, key_b), offsetof(b2l_seq_latent_attn_args, sink), "
                    "offsetof(b2l_seq_latent_attn_args, scale), offsetof(b2l_seq_latent_attn_args, act_dtype));return 0;}\n")
    exe = tmp_path / "layout"
    subprocess.run(["gcc", "-I", os.path.join(ROOT, "include"), str(prog), "-o", str(exe)], check=True)
    out = [int(v) for v in subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split()]
    A = S.LatentAttnArgs
    assert out == [C.sizeof(A), A.key_b.offset, A.sink.offset, A.scale.offset, A.act_dtype.offset]


def test_oracle_retention_state_carries():
    torch.manual_seed(3)
    m = {"heads": 2, "dim": 6, "vdim": 4, "decay": [0.9, 1.0], "rot": {"base": 20.0, "dims": 4}}
    W = {"q": torch.randn(12, 8), "k": torch.randn(12, 8), "v": torch.randn(8, 8), "g": torch.randn(8, 8), "o": torch.randn(8, 8)}
    W = {k: v.double() for k, v in W.items()}
    h = torch.randn(11, 8, dtype=torch.float64)
    whole, S_end = O.retention(h, W, "", m, 1e-6)
    a, S_mid = O.retention(h[:4], W, "", m, 1e-6)
    b, S_end2 = O.retention(h[4:], W, "", m, 1e-6, state=S_mid, pos0=4)
    assert torch.allclose(torch.cat([a, b]), whole, atol=1e-12) and torch.allclose(S_end, S_end2, atol=1e-12)
