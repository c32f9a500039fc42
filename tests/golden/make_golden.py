"""Generate golden vectors by RUNNING the reference's own CPU implementation (ref_ctct.py).

Usage (only where the reference checkout is available; the result is committed):

    python tests/golden/make_golden.py [/path/to/reference]

For every case the reference's four lattice functions (ref_fw_simple, ref_bw_simple,
ref_fw_shift, ref_bw_shift) are executed on seeded inputs and their tables and
log-likelihoods are stored; for cases without adjacent repeated labels the gradient of
-log-likelihood w.r.t. the full-vocabulary log-probs is taken by autograd through
ref_bw_shift (the only variant autograd can differentiate).  collect_units and
collect_separate outputs pin the gathers.  Nothing here is re-implemented: the numbers in
ctct_ref_golden.npz are outputs of the reference code.
"""
import os
import sys

import numpy as np
import torch

if len(sys.argv) < 2 and "WARP_CTCT_REFERENCE" not in os.environ:
    raise SystemExit("usage: python make_golden.py <checkout of maxwellzh/warp-ctct>  (or set WARP_CTCT_REFERENCE)")
REF = sys.argv[1] if len(sys.argv) > 1 else os.environ["WARP_CTCT_REFERENCE"]
sys.path.insert(0, REF)
import ref_ctct as R  # noqa: E402

OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "ctct_ref_golden.npz")
blob = {}
names = []


def add_case(name, lp, ys, want_autograd=True):
    lp = lp.float().contiguous()
    ys = ys.long()
    names.append(name)
    blob[f"{name}/lp"] = lp.numpy()
    blob[f"{name}/ys"] = ys.numpy().astype(np.int32)
    for key, fn in (("fw_simple", R.ref_fw_simple), ("bw_simple", R.ref_bw_simple),
                    ("fw_shift", R.ref_fw_shift), ("bw_shift", R.ref_bw_shift)):
        tab, ll = fn(lp, ys)
        blob[f"{name}/{key}"] = tab.numpy().astype(np.float32)
        blob[f"{name}/{key}_ll"] = np.float32(ll.item())
    blob[f"{name}/units"] = R.collect_units(lp[None], ys[None])[0].numpy()
    has_repeat = bool((ys[1:] == ys[:-1]).any())
    if want_autograd and not has_repeat:
        x = lp.clone().requires_grad_(True)
        (-R.ref_bw_shift(x, ys)[1]).backward()
        assert not torch.isnan(x.grad).any()
        blob[f"{name}/grad"] = x.grad.numpy()


# the reference's own printed demo (ref_ctct.py:233-255): seed 1, T,U,V = 5,2,4
torch.manual_seed(1)
T, U, V = 5, 2, 4
lp = torch.randn(T, U + 1, V).log_softmax(dim=-1)
ys = torch.randint(1, V, (U,))
add_case("demo", lp, ys)

# first benchmark configuration: B=2, T=16, U+1=5, V=8, labels in [1,7], full lengths
gen = torch.Generator().manual_seed(1000)
for n in range(2):
    lp = torch.randn(16, 5, 8, generator=gen).log_softmax(-1)
    ys = torch.randint(1, 8, (4,), generator=gen)
    add_case(f"cfg1_{n}", lp, ys)

# edge shapes: T == U (band of width 1), single label, single frame, repeats
gen = torch.Generator().manual_seed(7)
edge = [(4, 4, 8, [1, 2, 3, 4]), (5, 1, 6, [2]), (2, 1, 4, [3]), (1, 1, 4, [1]), (3, 2, 5, [4, 2]),
        (12, 4, 8, [3, 3, 5, 5]), (9, 3, 6, [2, 2, 2]), (20, 6, 11, [1, 7, 7, 3, 10, 1]),
        (33, 9, 16, None), (40, 17, 32, None)]
for k, (T, U, V, y) in enumerate(edge):
    lp = (1.5 * torch.randn(T, U + 1, V, generator=gen)).log_softmax(-1)
    ys = torch.tensor(y) if y is not None else torch.randint(1, V, (U,), generator=gen)
    add_case(f"edge{k}", lp, ys, want_autograd=(T * U <= 400))

# collect_separate (ref_ctct.py:206-220) on a small batch
gen = torch.Generator().manual_seed(11)
f = torch.randn(2, 7, 9, generator=gen)
g = torch.randn(2, 4, 9, generator=gen)
ys = torch.randint(1, 9, (2, 3), generator=gen)
cf, cg = R.collect_separate(f, g, ys)
blob["sep/f"], blob["sep/g"], blob["sep/ys"] = f.numpy(), g.numpy(), ys.numpy().astype(np.int32)
blob["sep/cf"], blob["sep/cg"] = cf.numpy(), cg.numpy()

blob["names"] = np.array(names)
np.savez_compressed(OUT, **blob)
print("wrote", OUT, os.path.getsize(OUT), "bytes;", len(names), "cases")
