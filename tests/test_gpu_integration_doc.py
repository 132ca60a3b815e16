"""Executes the ctypes binding example of INTEGRATION.md as it is written there, so that the document
cannot drift from include/paro_b200.h, and checks its result against the oracle."""
import os
import re

import pytest
import torch

from oracle import paro_oracle as po
from paroatten_b200 import _lib

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_the_documented_binding_runs_and_is_correct():
    with open(os.path.join(ROOT, "INTEGRATION.md")) as f:
        text = f.read()
    section = text[text.index("## 2. Binding the C ABI directly"):text.index("## 3. Build")]
    blocks = re.findall(r"```python\n(.*?)```", section, flags=re.S)
    assert len(blocks) == 1
    _lib.lib()                                   # builds the library if needed
    B, H, N, D = 2, 3, 1000, 128
    q, k, v, _ = po.make_inputs(B, H, N, D, torch.bfloat16, seed=77)
    mask = po.make_mask(H, (N + 63) // 64, 0.5, seed=77)
    env = {"q": q.cuda(), "k": k.cuda(), "v": v.cuda(), "mask": mask.cuda(), "LIB": _lib.LIB_PATH}
    exec(compile(blocks[0], "INTEGRATION.md", "exec"), env)
    want, want_lse = po.paro_attention(q, k, v, [0] * H, mask, (1, 1, N), return_lse=True)
    out, lse = env["out"].cpu(), env["lse"].cpu()
    assert po.cosine_per_head(out, want).min().item() >= 0.9995
    assert po.rel_l1_per_head(out, want).max().item() <= 1e-2
    assert (lse - want_lse).abs().max().item() < 2e-3
    assert int(env["redo"][0]) == 0 and int(env["status"][0]) == 0
