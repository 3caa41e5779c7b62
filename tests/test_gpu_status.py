"""The time-out reporting path of the kernels' bounded waits, exercised without faulting or hanging anything:
a self-test kernel waits one millisecond on a barrier that nothing completes, gives up and reports through the
status word; launches that follow are unaffected."""
import math

import pytest
import torch

import oracle
from parity_util import close, cpu_quant, gen

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def qfa():
    import quant_flash_attn_b200 as m
    from quant_flash_attn_b200 import _lib
    _lib.load()
    return m


def test_wait_timeout_is_reported_and_later_launches_are_healthy(qfa):
    from quant_flash_attn_b200 import _lib
    lib = _lib.load()
    dev = torch.device("cuda", torch.cuda.current_device())
    stream = torch.cuda.current_stream().cuda_stream
    # a device-memory status word, as a C caller would pass
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    assert lib.qfa_selftest_wait_timeout(0, status.data_ptr(), stream) == -3          # budget out of range
    assert lib.qfa_selftest_wait_timeout(10 ** 9, status.data_ptr(), stream) == -3
    assert lib.qfa_selftest_wait_timeout(1000, None, stream) == -1
    t0 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0[0].record()
    assert lib.qfa_selftest_wait_timeout(1_000_000, status.data_ptr(), stream) == 0   # 1 ms
    t0[1].record()
    torch.cuda.synchronize()
    assert int(status.item()) == 1 and lib.qfa_strerror(1) == b"a bounded barrier wait inside a kernel ran out"
    assert 0.9 <= t0[0].elapsed_time(t0[1]) < 50.0                                    # gave up after the budget, promptly

    # the same through the package's own status word (pinned host memory the GPU writes directly): the next
    # operator call on the device reports it once, without anybody having synchronised for it
    word = _lib.status_word(dev)
    assert lib.qfa_selftest_wait_timeout(1_000_000, word.data_ptr(), stream) == 0
    torch.cuda.synchronize()
    q, k, v = (gen((1, 2, 300, 128), torch.bfloat16, s) for s in (1, 2, 3))
    qq, kq, vq = qfa.quantize_qkv(q.cuda(), k.cuda(), v.cuda())
    sm = 1.0 / math.sqrt(128)
    with pytest.raises(RuntimeError, match="bounded barrier wait"):
        qfa.int8_attention_forward(qq, kq, vq, True, sm, torch.bfloat16)
    assert int(word[0]) == 0                                                          # reported once, then cleared

    # launches after a time-out run normally: the forward kernels share the device-side abort word with the
    # self-test kernel, and every launch draws a fresh epoch
    o, lse = qfa.int8_attention_forward(qq, kq, vq, True, sm, torch.bfloat16)
    qfa.check_kernel_status()
    o_ref, lse_ref, _ = oracle.int8_mode_forward(q, k, v, True, sm, quant=tuple(cpu_quant(t) for t in (qq, kq, vq)),
                                                 round_output=False)
    close(o, o_ref, what="forward after a reported time-out")
    assert (lse.cpu() - lse_ref).abs().max().item() <= 2e-3
    # short-query kernels (bulk-copy ring with bounded waits) as well
    qs = gen((2, 2, 16, 128), torch.float16, 4).cuda()
    kv = gen((2, 2, 500, 128), torch.float16, 5).cuda()
    kvq = qfa.asymmetric_quant_per_token(kv)
    out = qfa.quant_flash_attn(qs, kv, kvq, sm)
    qfa.check_kernel_status()
    o2, _ = oracle.ref_mode_forward(qs.cpu(), *(t.cpu() for t in kvq), sm, round_output=False)
    close(out, o2, what="short-query forward after a reported time-out")
