"""A bounded device-side wait that runs out, on one GPU and without any fault: a sharded engine (rank 0 of 2) is given
a loopback exchange in which the other rank's share never arrives.  Every exchange wait then reaches its (shortened)
bound, the kernels carry on, the step finishes, and the host reads PI_ERR_TIMEOUT from the status word.  After the shares
are filled in from the host the same engine runs clean steps again: the context was never lost."""
import numpy as np
import pytest

from powerinfer_b200 import synth

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def test_exchange_wait_runs_out_and_the_engine_stays_usable():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from powerinfer_b200 import engine
    from powerinfer_b200._lib import lib
    spec = synth.ModelSpec(arch=synth.ARCH_LLAMA, wtype=synth.Q4_0, n_layer=2, d=512, n_ff=2048, n_head=4, n_head_kv=2, rank=64,
                           firing=0.15, seed=41)
    eng = engine.DecodeEngine(spec, synth.build_model(spec), max_batch=1, n_ranks=2, rank=0)
    eng.setup_exchange_loopback()
    eng.set_wait_cycles(2_000_000)                 # about a millisecond per wait instead of a second
    for step in range(3):                          # plain launch, graph capture, graph replay
        eng.decode([7], [step])
        rc = lib.pi_engine_status(eng.handle, eng.st)
        assert rc == 5, (step, rc, lib.pi_last_error())        # PI_ERR_TIMEOUT
        assert b"exchange" in lib.pi_last_error()
    assert lib.pi_engine_status(eng.handle, eng.st) == 0       # reported once, then cleared
    eng.fill_peer_shares()
    logits, amax = eng.decode([7], [3])
    eng.status()                                               # clean
    assert np.isfinite(logits).all() and int(amax[0]) == int(logits[0].argmax())
    eng.close()
