"""The exchange of output slices between GPUs over peer memory (sgk_peer_*, sgk_exchange_*): two
processes, one per GPU, each stores its slice into the other's rows and waits for the other's flag.
Needs two GPUs; skipped on one. The waits are bounded on the device and on the host; the last
phase makes one of them run out (a peer that stays alive but stops joining) and checks the report."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu


def _gpus():
    import torch
    return torch.cuda.device_count()


def test_two_ranks_exchange_slices_over_peer_memory(tmp_path):
    if _gpus() < 2:
        pytest.skip("needs two GPUs")
    helper = os.path.join(os.path.dirname(os.path.abspath(__file__)), "helpers", "exchange_rank.py")
    procs = [subprocess.Popen([sys.executable, helper, str(r), "2", str(tmp_path)], stdout=subprocess.PIPE,
                              stderr=subprocess.PIPE, text=True) for r in range(2)]
    outs = []
    for p in procs:
        try:
            outs.append(p.communicate(timeout=300))
        except subprocess.TimeoutExpired:
            p.kill()
            outs.append(p.communicate())
    for p, (out, err) in zip(procs, outs):
        assert p.returncode == 0 and "OK" in out, err[-2000:]
    # the rank whose peer stopped joining saw its bounded wait run out and went on
    assert "TIMEOUT-REPORTED" in outs[0][0] and "TIMEOUT-REPORTED" not in outs[1][0]


def test_exchange_rejects_bad_arguments():
    import saragossa_b200 as sg
    st = sg.DecodeResidentState(0)
    with pytest.raises(sg.InferError):
        st.exchange(0, 1)          # one rank has nobody to exchange with
    with pytest.raises(sg.InferError):
        st.exchange(3, 2)
    ex = st.exchange(0, 2)
    buf = st.alloc(1024)
    with pytest.raises(sg.InferError) as err:
        ex.enqueue(buf.ptr, [0, buf.ptr], 0, 64)   # peer 1 not connected
    assert err.value.kind == "Config"
    with pytest.raises(sg.InferError):
        ex.connect(0, ex.handle)   # own rank
    with pytest.raises(sg.InferError):
        ex.enqueue(buf.ptr, [0, buf.ptr], 2, 64)   # offset not a multiple of 4
    ex.close()
    st.close()
