"""A checkpoint written by the reference library (whole ``state_dict()``, pickled configuration
objects in ``param_groups`` included) loads into this framework in a process that does not have the
reference installed, and training continues bit for bit like the reference itself continues."""

import os
import subprocess
import sys
import textwrap

import pytest
import torch

from ref_oracle import REF_DIR, reference_available

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

COMMON = textwrap.dedent(
    """
    import sys, torch
    def model():
        torch.manual_seed(0)
        return torch.nn.Sequential(torch.nn.Linear(10, 12), torch.nn.ReLU(), torch.nn.Linear(12, 6, bias=False), torch.nn.ReLU(), torch.nn.Linear(6, 3))
    def batches(n, seed):
        g = torch.Generator().manual_seed(seed)
        return [(torch.randn(16, 10, generator=g), torch.randint(0, 3, (16,), generator=g)) for _ in range(n)]
    def make(lib, params):
        return lib.DistributedShampoo(
            params, lr=0.01, betas=(0.9, 0.999), epsilon=1e-8, max_preconditioner_dim=8, precondition_frequency=2,
            start_preconditioning_step=2, weight_decay=1e-3, grafting_config=lib.AdamPreconditionerConfig(beta2=0.999),
            preconditioner_config=lib.RootInvShampooPreconditionerConfig(),
        )
    def train(m, opt, data):
        for x, y in data:
            opt.zero_grad()
            torch.nn.functional.cross_entropy(m(x), y).backward()
            opt.step()
    """
)


@pytest.mark.skipif(not reference_available(), reason="reference library is not installed under baseline/_ref")
def test_reference_checkpoint_loads_without_the_reference_installed(tmp_path):
    ckpt, ref_final, our_final = (str(tmp_path / n) for n in ("ckpt.pt", "ref.pt", "ours.pt"))
    writer = COMMON + textwrap.dedent(
        f"""
        sys.path.insert(0, {REF_DIR!r})
        import distributed_shampoo as lib
        m = model(); opt = make(lib, m.parameters())
        train(m, opt, batches(5, 1))
        torch.save({{"model": m.state_dict(), "optim": opt.state_dict()}}, {ckpt!r})
        train(m, opt, batches(4, 2))
        torch.save([p.detach() for p in m.parameters()], {ref_final!r})
        """
    )
    reader = COMMON + textwrap.dedent(
        f"""
        sys.path.insert(0, {REPO!r})
        import importlib.util
        assert importlib.util.find_spec("distributed_shampoo") is None  # the reference is not importable here
        import optimizers_b200 as lib
        from optimizers_b200.compat import install_reference_aliases
        assert install_reference_aliases()
        blob = torch.load({ckpt!r}, weights_only=False)
        group = blob["optim"]["param_groups"][0]
        assert type(group["grafting_config"]) is lib.AdamPreconditionerConfig
        assert type(group["preconditioner_config"]) is lib.RootInvShampooPreconditionerConfig
        m = model()
        with torch.no_grad():
            for p in m.parameters():
                p.mul_(0.0)
        opt = make(lib, m.parameters())
        m.load_state_dict(blob["model"]); opt.load_state_dict(blob["optim"])
        train(m, opt, batches(4, 2))
        torch.save([p.detach() for p in m.parameters()], {our_final!r})
        """
    )
    env = {k: v for k, v in os.environ.items() if k != "PYTHONPATH"}
    for script in (writer, reader):
        res = subprocess.run([sys.executable, "-c", script], env=env, capture_output=True, text=True, timeout=600, cwd=str(tmp_path))
        assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    for a, b in zip(torch.load(ref_final), torch.load(our_final)):
        assert torch.equal(a, b), (a - b).abs().max()
