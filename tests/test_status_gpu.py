"""The failure path of the kernels' bounded waits, without faulting a device.

Host form: a code written into the status word from the host must surface, with what it means, through
``ModelRunner.check_device_status``, ``LLM.generate`` and ``bin/trace_run`` (non-zero exit), and go away with a
reset.  Device form: one CTA waits, with the products' own wait cut down to a thousand polls, on an mbarrier
that nobody arrives at; it must give up, record its code, free its tensor memory and return, and a product
launched right after it must be right.  (The reference's waits are unbounded spins:
crates/kernels/cuda/umma.cuh:127-137; its engine ends every live request on a step error:
crates/core/src/engine.rs:468-475.)
"""
import importlib.machinery
import importlib.util
import io
import json
import os
import sys

import pytest
import torch

import helpers as H

pytestmark = pytest.mark.gpu

CODES = [1, 2, 3, 11, 12, 13, 14, 15, 16, 21, 22]


@pytest.fixture(scope="module")
def model_dir(tmp_path_factory):
    d = tmp_path_factory.mktemp("status")
    return H.make_model_dir(str(d), H.TINY_D, *H.INIT["D"], torch.bfloat16)


def poke(code: int) -> None:
    from dinfer_b200.kernels import gemm_ops
    gemm_ops._state(torch.device("cuda", torch.cuda.current_device()))["status"].fill_(code)


def test_a_status_written_from_the_host_surfaces_with_its_meaning(model_dir):
    from dinfer_b200 import LLM, SamplingParams
    from dinfer_b200.kernels import gemm_ops
    from dinfer_b200.kernels.lib import KernelError
    llm = LLM(model_dir, dtype="bfloat16", max_model_len=64, max_num_seqs=2, max_num_batched_tokens=32, num_blocks=8)
    r = llm.runner
    r.check_device_status()                                  # fine to begin with
    for code in CODES:
        poke(code)
        with pytest.raises(KernelError) as e:
            r.check_device_status()
        msg = str(e.value)
        assert f"status {code}" in msg and gemm_ops.STATUS_MEANING[code] in msg
        kind = "matrix product" if code < 10 else ("prompt attention" if code < 20 else "decode attention")
        assert kind in msg
        with pytest.raises(KernelError):                     # it stays reported until it is reset
            r.check_device_status()
        assert r.reset_device_status() == code
        r.check_device_status()
    poke(99)
    with pytest.raises(KernelError, match="unknown code"):
        r.check_device_status()
    r.reset_device_status()
    # generation ends with the check
    sp = SamplingParams(temperature=0.0, max_tokens=3, ignore_eos=True)
    assert len(llm.generate([[1, 2, 3]], sp)[0].output_ids) == 3
    poke(13)
    with pytest.raises(KernelError, match="softmax warps' P tile"):
        llm.generate([[4, 5, 6]], sp)
    assert r.reset_device_status() == 13
    assert len(llm.generate([[1, 2, 3]], sp)[0].output_ids) == 3


def test_trace_run_stops_with_an_error_when_a_kernel_reported_a_fault(model_dir, tmp_path, monkeypatch, capsys):
    path = os.path.join(H.ROOT, "bin", "trace_run")
    loader = importlib.machinery.SourceFileLoader("trace_run_under_test", path)
    spec = importlib.util.spec_from_loader(loader.name, loader)
    mod = importlib.util.module_from_spec(spec)
    loader.exec_module(mod)
    from dinfer_b200.engine.runner import ModelRunner
    from dinfer_b200.kernels import gemm_ops
    inner = ModelRunner.step
    calls = []

    def step(self, entries, *a, **kw):
        out = inner(self, entries, *a, **kw)
        calls.append(len(entries))
        if len(calls) == 2:
            poke(22)                                         # as if the second step's decode attention had given up
        return out

    monkeypatch.setattr(ModelRunner, "step", step)
    lines = [json.dumps({"step": i, "entries": [{"id": "a", "tokens": t, "want": [0]}], "end": []})
             for i, t in enumerate([[1, 2, 3], [4], [5]])]
    monkeypatch.setattr(sys, "stdin", io.StringIO("\n".join(lines) + "\n"))
    monkeypatch.setattr(sys, "argv", ["trace_run", "--model", model_dir, "--dtype", "bfloat16",
                                      "--out", str(tmp_path / "o"), "--max-tokens", "64"])
    try:
        rc = mod.main()
    finally:
        gemm_ops.reset_status()
    out = capsys.readouterr()
    assert rc != 0 and len(calls) == 2                       # the third step never ran
    assert "done 0" in out.out and "done 1" not in out.out
    assert "status 22" in out.err and "decode attention" in out.err


def test_a_wait_that_runs_out_returns_its_code_and_the_device_stays_usable():
    from dinfer_b200.kernels import gemm_ops as G
    from dinfer_b200.kernels.lib import KernelError
    G.reset_status()
    g = torch.Generator().manual_seed(3)
    x = torch.randn(8, 512, generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn(384, 512, generator=g) / 22.0).to(torch.bfloat16).cuda()
    want = x.float() @ w.float().T
    for polls in (1000, 1, 4096):
        assert G.wait_probe(polls) == 2                      # gave up, said so, and came back
        with pytest.raises(KernelError, match="status 2"):
            G.check_status()
        assert G.reset_status() == 2
        out = torch.full((8, 384), float("nan"), dtype=torch.bfloat16, device="cuda")
        G.gemm_tc(x, w, out)                                 # tensor memory was freed: the next product allocates and runs
        big = torch.full((600, 384), float("nan"), dtype=torch.bfloat16, device="cuda")
        G.gemm_tc(x.repeat(75, 1), w, big)                   # and the two-SM kernel, which takes all 512 columns
        torch.cuda.synchronize()
        assert float((out.float() - want).abs().max()) < 2e-2 * float(want.abs().max())
        assert float((big[-8:].float() - want).abs().max()) < 2e-2 * float(want.abs().max())
        G.check_status()
    with pytest.raises(KernelError, match="polls"):
        G.wait_probe(0)
