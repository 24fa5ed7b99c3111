"""A bounded device-side wait that actually runs out — on ONE GPU, without hanging anything.

The kernels that exchange data with other GPUs wait for flags or tagged words that a peer
writes.  Every such wait has a limit (about a second of SM cycles; the launchers pass it to
the kernel).  Here the limit is shortened to a few milliseconds through the debug knob and the
"peer" is a local zero-filled buffer that nobody ever signals: the kernel must return by
itself, the status word must name the wait that gave up, `b200q_check_status` must turn it into
`B200Q_ERR_DEVICE_TIMEOUT` and clear it, the rank's call counter must have moved on so that
the NEXT call pairs up with its peers again, and ordinary kernels must be unaffected.

This replaces the reference's failure behaviour for the path — a failing extension call is
swallowed and the layer silently computes something else (nanovllm/quantization/cuda.py:347-356,
493-503) — by an error the caller sees.  Nothing here faults, traps or spins without a limit.
"""
import ctypes
import time

import pytest
import torch

from oracle import quant_linear_oracle as O
from gpu_util import bits, knobs
from tiny_vllm_b200 import _lib
from tiny_vllm_b200.quantization.cuda import apply_w8a8_linear

pytestmark = pytest.mark.gpu

WAIT_CYCLES = 4_000_000          # about 2 ms at 2 GHz
# 32-bit slots of a flag pad (two-shot / pull kernels) and of the tagged-word control block
SLOT_EPOCH, SLOT_A, SLOT_B = 0, 16, 32


def ptr_array(*tensors):
    return (ctypes.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])


def stream():
    return torch.cuda.current_stream().cuda_stream


def expect_timeout(code):
    """The launch returned; the kernel must end by itself within the shortened limit."""
    t0 = time.perf_counter()
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 2.0, "kernel did not give up within the shortened limit"
    word = ctypes.c_int(0)
    rc = _lib.lib().b200q_check_status(ctypes.byref(word))
    assert rc == _lib.ERR_DEVICE_TIMEOUT and word.value == code, (rc, hex(word.value))
    assert _lib.lib().b200q_strerror(rc).decode() == "a bounded device-side wait gave up"
    with pytest.raises(_lib.B200QError):
        # the word was cleared by the read above: raise it again by hand to check the wrapper
        raise _lib.B200QError(rc, "check")
    assert _lib.lib().b200q_check_status(None) == _lib.OK          # cleared by the first read


def ordinary_gemm_still_exact():
    q, s = O.make_weight(256, 512, seed=4)
    x = O.make_activation(130, 512, seed=4)
    xq, a_s = O.quantize_per_row_dynamic(x)
    y = apply_w8a8_linear(xq.cuda(), a_s.cuda(), q.cuda(), s.cuda(), out_dtype=torch.bfloat16)
    expect = O.w8a8_native_epilogue(O.w8a8_int32_accumulators(xq, q), a_s, s, None, torch.bfloat16)
    assert torch.equal(bits(y.cpu()), bits(expect))


@pytest.mark.parametrize("variant,code", [("two_shot", 0x501), ("pull", 0x503)])
def test_flag_wait_runs_out_and_the_next_call_pairs_up_again(variant, code, oracle_c_lib):
    L = _lib.lib()
    n = 1 << 15
    g = torch.Generator().manual_seed(7)
    mine = torch.randn(n, generator=g).to(torch.bfloat16)
    peer = torch.randn(n, generator=g).to(torch.bfloat16)
    buf0, buf1 = mine.cuda(), peer.cuda()           # "rank 1" is a local buffer nobody works on
    pad0 = torch.zeros(1024, dtype=torch.int32, device="cuda")
    pad1 = torch.zeros(1024, dtype=torch.int32, device="cuda")
    out = torch.empty(n, dtype=torch.bfloat16, device="cuda")
    bufs, pads = ptr_array(buf0, buf1), ptr_array(pad0, pad1)

    def call():
        if variant == "two_shot":
            return L.b200q_tp_allreduce(bufs, pads, 0, 2, n, _lib.DTYPE_BF16, stream())
        return L.b200q_tp_allreduce_pull(bufs, pads, out.data_ptr(), 0, 2, n, _lib.DTYPE_BF16, stream())

    with knobs(WAIT_CYCLES=WAIT_CYCLES):
        assert call() == _lib.OK
        expect_timeout(code)
        # nothing was reduced, and the rank's call counter moved on to 1
        assert torch.equal(bits(buf0.cpu()), bits(mine))
        assert int(pad0[SLOT_EPOCH].item()) == 1
        ordinary_gemm_still_exact()
        # second call = call number 2: this time the "peer" has announced itself (the host plays
        # its part by writing the two flags it would have written), so the call goes through
        pad0[SLOT_A + 1] = 2
        pad0[SLOT_B + 1] = 2
        torch.cuda.synchronize()
        assert call() == _lib.OK
        torch.cuda.synchronize()
        assert L.b200q_check_status(None) == _lib.OK
    total = (mine.float() + peer.float()).to(torch.bfloat16)
    if variant == "two_shot":        # rank 0 reduces the first half and writes it to both buffers
        half = n // 2
        assert torch.equal(bits(buf0[:half].cpu()), bits(total[:half]))
        assert torch.equal(bits(buf1[:half].cpu()), bits(total[:half]))
        assert torch.equal(bits(buf0[half:].cpu()), bits(mine[half:]))
    else:
        assert torch.equal(bits(out.cpu()), bits(total))
    assert int(pad0[SLOT_EPOCH].item()) == 2


def test_tagged_word_wait_runs_out_in_the_fused_decode_kernel(oracle_c_lib):
    # b200q_w8a8_gemm_allreduce: the GEMM's CTAs push their partial tiles and poll for the
    # peer's words; the peer never writes -> status 0x601; then call number 2 with the peer's
    # words already in place (written by the host) completes with the right sum
    L = _lib.lib()
    M, N, K = 16, 256, 512
    q, s = O.make_weight(N, K, seed=11)
    x = O.make_activation(M, K, seed=11)
    xq, a_s = O.quantize_per_row_dynamic(x)
    part = O.w8a8_native_epilogue(O.w8a8_int32_accumulators(xq, q), a_s, s, None, torch.bfloat16)
    recv_bytes = 1 << 20
    recv0 = torch.zeros(recv_bytes // 4, dtype=torch.int32, device="cuda")
    recv1 = torch.zeros(recv_bytes // 4, dtype=torch.int32, device="cuda")
    ctl0 = torch.zeros(64, dtype=torch.int32, device="cuda")
    ctl1 = torch.zeros(64, dtype=torch.int32, device="cuda")
    y = torch.zeros(M, N, dtype=torch.bfloat16, device="cuda")
    dev = [t.cuda() for t in (xq, a_s, q, s)]
    recv, ctl = ptr_array(recv0, recv1), ptr_array(ctl0, ctl1)

    def call():
        return L.b200q_w8a8_gemm_allreduce(dev[0].data_ptr(), dev[1].data_ptr(), dev[2].data_ptr(),
                                           dev[3].data_ptr(), None, y.data_ptr(), M, N, K,
                                           _lib.DTYPE_BF16, recv, ctl, recv_bytes, 0, 2, stream())

    with knobs(WAIT_CYCLES=WAIT_CYCLES):
        assert call() == _lib.OK
        expect_timeout(0x601)
        assert int(ctl0[0].item()) == 1                    # call counter in step
        ordinary_gemm_still_exact()
        # call number 2 uses parity half 0 of the receive area; rank 1's slot follows rank 0's.
        # A word is {two 16-bit values, call number}.
        peer_part = (part.float() * 0.5).to(torch.bfloat16)
        words = peer_part.contiguous().view(torch.int32).view(M, N // 2)
        tagged = torch.stack([words, torch.full_like(words, 2)], dim=-1).reshape(-1)
        slot_words = M * (N // 2)
        recv0[2 * slot_words:2 * slot_words + tagged.numel()] = tagged.cuda()
        torch.cuda.synchronize()
        assert call() == _lib.OK
        torch.cuda.synchronize()
        assert L.b200q_check_status(None) == _lib.OK
    expect = (part.float() + peer_part.float()).to(torch.bfloat16)
    assert torch.equal(bits(y.cpu()), bits(expect))
    assert int(ctl0[0].item()) == 2


def test_tagged_word_wait_runs_out_in_the_small_allreduce():
    L = _lib.lib()
    n = 4096
    x = torch.randn(n, generator=torch.Generator().manual_seed(3)).to(torch.bfloat16).cuda()
    y = torch.zeros_like(x)
    recv_bytes = 1 << 20
    recv0 = torch.zeros(recv_bytes // 4, dtype=torch.int32, device="cuda")
    recv1 = torch.zeros(recv_bytes // 4, dtype=torch.int32, device="cuda")
    ctl0 = torch.zeros(64, dtype=torch.int32, device="cuda")
    ctl1 = torch.zeros(64, dtype=torch.int32, device="cuda")
    with knobs(WAIT_CYCLES=WAIT_CYCLES):
        rc = L.b200q_tp_allreduce_small(x.data_ptr(), y.data_ptr(), n, _lib.DTYPE_BF16,
                                        ptr_array(recv0, recv1), ptr_array(ctl0, ctl1), recv_bytes,
                                        0, 2, stream())
        assert rc == _lib.OK
        expect_timeout(0x602)
    assert int(ctl0[0].item()) == 1
    assert not y.any()                                     # nothing was written without the peer


def test_default_limit_is_untouched_by_other_threads_knobs():
    # knobs are per thread: a setting made here is invisible to a thread that never set one
    import threading
    L = _lib.lib()
    seen = {}
    with knobs(WAIT_CYCLES=123, NO_PAIR=1):
        def other():
            seen["path"] = L.b200q_select_path(_lib.OP_W8A8, 8192, 4096, 1024).decode()
        t = threading.Thread(target=other)
        t.start()
        t.join()
        assert L.b200q_select_path(_lib.OP_W8A8, 8192, 4096, 1024).decode() == "umma_i8_tokens128"
    assert seen["path"] == "umma_i8_pair_tokens256"
