"""Helpers shared by the tests that use the committed golden fixtures."""
import hashlib
from pathlib import Path

import numpy as np
import torch

from pypto_b200 import inputs as gen

GOLDEN = Path(__file__).resolve().parent / "golden"


def sha(t: torch.Tensor) -> str:
    return hashlib.sha256(t.contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()


def from_np_bf16(a) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a)).view(torch.bfloat16)


def load_case(name: str, **kw):
    """Regenerate the fixture's inputs from its seed and check them against the stored digests."""
    z = np.load(GOLDEN / f"{name}.npz")
    act_seq = [int(x) for x in z["act_seq"]]
    s1 = int(z["s1"])
    if name.startswith("li_nonquant_"):
        d = gen.make_nonquant_inputs(act_seq, s1=s1, seed=int(z["seed"]), with_attention=False)
    elif name.startswith("li_"):
        d = gen.make_inputs(act_seq, s1=s1, seed=int(z["seed"]), scale_dtype=getattr(torch, str(z["scale_dtype"])),
                            with_attention=False)
    else:
        d = gen.make_inputs(act_seq, s1=s1, seed=int(z["seed"]), with_indexer=False, with_topk=True)
    want = dict(h.split("=") for h in z["hashes"])
    got = {k: sha(v) for k, v in d.tensors().items()}
    assert got == want, f"regenerated inputs of {name} differ from the ones the fixture was made with"
    return d, z


PROLOG_CASES = ["prolog_mtp", "prolog_single"]
PROLOG_HEADS = (0, 37, 127)  # heads of q_nope the fixture keeps in full


def load_prolog_case(name: str):
    z = np.load(GOLDEN / f"{name}.npz")
    p = gen.make_prolog_inputs([int(x) for x in z["act_seq"]], s1=int(z["s1"]), seed=int(z["seed"]))
    want = dict(h.split("=") for h in z["hashes"])
    got = {k: sha(v) for k, v in p.items() if isinstance(v, torch.Tensor)}
    assert got == want, f"regenerated inputs of {name} differ from the ones the fixture was made with"
    return p, z


PROLOG_NONQUANT_CASES = ["prolog_nonquant_single", "prolog_nonquant_mtp"]


def load_prolog_nonquant_case(name: str):
    z = np.load(GOLDEN / f"{name}.npz")
    p = gen.make_prolog_nonquant_inputs([int(x) for x in z["act_seq"]], s1=int(z["s1"]), seed=int(z["seed"]))
    want = dict(h.split("=") for h in z["hashes"])
    got = {k: sha(v) for k, v in p.items() if isinstance(v, torch.Tensor)}
    assert got == want, f"regenerated inputs of {name} differ from the ones the fixture was made with"
    return p, z


LI_CASES = ["li_ragged_f32", "li_mtp_f16", "li_short_f16"]
NONQUANT_CASES = ["li_nonquant_mtp", "li_nonquant_ragged"]
SFA_CASES = ["sfa_ragged_mtp", "sfa_single"]


def mask_empty_rows(want: torch.Tensor, d) -> torch.Tensor:
    """Zero the rows of a reference attention output whose query token sees no key: the
    reference golden stores a stale value there (see test_degenerate_rows)."""
    want = want.clone().reshape(d.b, d.s1, *want.shape[-2:])
    for bi, s in enumerate(d.act_seq):
        for i in range(d.s1):
            if s - d.s1 + 1 + i <= 0:
                want[bi, i] = 0
    return want
