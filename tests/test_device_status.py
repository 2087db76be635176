"""The path a kernel's bounded wait takes when it runs out: a code in a host-visible word, raised
by `Engine.check_device_status()` after the next synchronisation.  The reference's analogue is a
failed buffer map that silently leaves the output untouched (gpu_backend.rs:534-540); here it is an
error with a text.  No kernel of the library is made to fail: the host-side test writes the codes
itself, and the GPU test runs the same `mbar_wait` + `report` on a barrier nothing arrives at, with a
limit of a few thousand polls."""
import pytest
import torch

from rust_inference_b200.kernels import tcgen05
from rust_inference_b200.kernels.ops import KernelError


def _bare_engine(dtype):
    from rust_inference_b200.engine.engine import Engine
    eng = Engine.__new__(Engine)                      # check_device_status reads the dtype only
    eng.dtype = dtype
    return eng


def test_every_code_raises_its_text_and_clears_the_word(monkeypatch):
    word = torch.zeros(1, dtype=torch.int32)
    monkeypatch.setattr(tcgen05, "_status", word)
    eng = _bare_engine(torch.bfloat16)
    eng.check_device_status()                         # nothing stored: nothing raised
    assert len(tcgen05.STATUS_TEXT) >= 12
    for code, text in tcgen05.STATUS_TEXT.items():
        word[0] = code
        with pytest.raises(KernelError) as e:
            eng.check_device_status()
        assert text in str(e.value)
        assert int(word[0]) == 0                      # cleared: the next check passes
        eng.check_device_status()
    word[0] = 99                                      # a code without a text still raises
    with pytest.raises(KernelError, match="code 99"):
        eng.check_device_status()


def test_a_32_bit_run_has_no_tensor_core_status(monkeypatch):
    word = torch.zeros(1, dtype=torch.int32)
    word[0] = 2
    monkeypatch.setattr(tcgen05, "_status", word)
    _bare_engine(torch.float32).check_device_status()  # the float32 path launches no kernel that reports there
    assert int(word[0]) == 2


@pytest.mark.gpu
def test_a_wait_that_runs_out_reports_and_the_device_goes_on(model_factory):
    from conftest import TOL, random_tokens, rel_err
    from rust_inference_b200.engine.engine import Engine
    model = model_factory("A", std=0.08)
    eng = Engine.from_pretrained(model.folder, dtype="bfloat16", max_tokens=256)
    torch.cuda.synchronize()
    eng.check_device_status()
    # a wait that succeeds leaves the word alone
    tcgen05.wait_probe(limit=2000, code=2, arrive_first=True)
    torch.cuda.synchronize()
    eng.check_device_status()
    # a wait on a barrier nothing arrives at: out of patience after 2,000 polls, code stored, kernel returns
    for code in (2, 13, 22):
        tcgen05.wait_probe(limit=2000, code=code)
        torch.cuda.synchronize()
        with pytest.raises(KernelError) as e:
            eng.check_device_status()
        assert tcgen05.STATUS_TEXT[code] in str(e.value)
        eng.check_device_status()                     # cleared
    with pytest.raises(KernelError, match="limit"):
        tcgen05.wait_probe(limit=0)
    # the context is as usable as before: an ordinary step still gives the plain logits
    toks = random_tokens(50, model.cfg["vocab_size"], seed=4)
    s = eng.alloc_slot()
    got = eng.step([s], [toks], "all")
    assert rel_err(got, model.plain_logits(toks)) <= TOL["bfloat16"]
    eng.check_device_status()
