"""The collectives layer (mcd_nccl_*) against a stand-in for NCCL: no GPU, no network, failures made on the host.

What is checked: results of the NCCL calls reach the caller as error codes with NCCL's own text in
mcd_last_error(); a call that stays in progress runs into the bounded poll, the communicator is aborted
(ncclCommAbort) and every later call on it fails at once instead of waiting again."""

import ctypes as C
import time

import pytest


@pytest.fixture
def fake(mc):
    lib = mc.lib()

    def install(failing_call=None, code=0, stay=False):
        assert lib.mcd_nccl_install_fake(failing_call.encode() if failing_call else None, code, int(stay)) == 0

    yield install
    lib.mcd_nccl_remove_fake()


def last(mc):
    return mc.lib().mcd_last_error().decode()


def test_a_healthy_communicator_runs_every_call(mc, fake):
    fake()
    uid = mc.Communicator.unique_id()
    assert len(uid) == 128
    comm = mc.Communicator(4, 2, uid, device=0, timeout_s=1.0)
    comm.broadcast(0x1000, 4096, root=0)
    comm.all_gather(0x1000, 0x2000, 1024)
    comm.wait()
    comm.broadcast(0x1000, 0, root=0)  # nothing to send is not an error
    assert mc.lib().mcd_nccl_fake_aborts() == 0
    comm.destroy()


@pytest.mark.parametrize("call,method", [("ncclBroadcast", "broadcast"), ("ncclAllGather", "all_gather")])
def test_an_nccl_error_reaches_the_caller_and_aborts_the_communicator(mc, fake, call, method):
    fake()
    comm = mc.Communicator(2, 0, mc.Communicator.unique_id(), device=0, timeout_s=1.0)
    fake(call, 3)  # ncclInternalError
    with pytest.raises(mc.McError, match=rf"{call}: internal error \(NCCL result 3\); the communicator was aborted"):
        if method == "broadcast":
            comm.broadcast(0x1000, 64)
        else:
            comm.all_gather(0x1000, 0x2000, 64)
    assert mc.lib().mcd_nccl_fake_aborts() == 1
    fake()  # NCCL is healthy again, the communicator is not
    with pytest.raises(mc.McError, match="aborted by an earlier failure"):
        comm.broadcast(0x1000, 64)
    comm.destroy()


def test_a_failing_init_returns_no_communicator(mc, fake):
    fake("ncclCommInitRankConfig", 5)  # ncclInvalidUsage
    with pytest.raises(mc.McError, match=r"ncclCommInitRankConfig: invalid usage"):
        mc.Communicator(2, 1, b"\0" * 128, device=0, timeout_s=1.0)
    fake()
    with pytest.raises(mc.McError, match="rank outside the world"):
        mc.Communicator(2, 2, b"\0" * 128, device=0)


def test_a_peer_that_never_joins_runs_into_the_timeout(mc, fake):
    """The stand-in stays 'in progress' for ever, as a communicator does whose peer never calls init."""
    fake(stay=True)
    t0 = time.perf_counter()
    with pytest.raises(mc.McError, match=r"ncclCommInitRankConfig did not complete within 0\.3 s \(rank 0 of 2\); the communicator was aborted"):
        mc.Communicator(2, 0, b"\0" * 128, device=0, timeout_s=0.3)
    waited = time.perf_counter() - t0
    assert 0.25 <= waited < 2.0
    assert mc.lib().mcd_nccl_fake_aborts() == 1


def test_a_collective_that_never_finishes_runs_into_the_timeout(mc, fake):
    fake()
    comm = mc.Communicator(2, 0, mc.Communicator.unique_id(), device=0, timeout_s=0.3)
    fake(stay=True)
    with pytest.raises(mc.McError, match=r"ncclBroadcast did not complete within 0\.3 s"):
        comm.broadcast(0x1000, 64)
    with pytest.raises(mc.McError, match="aborted by an earlier failure"):
        comm.wait()
    comm.destroy()


def test_an_asynchronous_error_is_seen_by_wait(mc, fake):
    fake()
    comm = mc.Communicator(8, 7, mc.Communicator.unique_id(), device=0, timeout_s=1.0)
    comm.broadcast(0x1000, 64)
    fake("ncclCommGetAsyncError", 6)  # ncclRemoteError: a peer died
    with pytest.raises(mc.McError, match=r"remote process exited.*the communicator was aborted"):
        comm.wait()
    comm.destroy()


def test_library_calls_fail_with_a_message_when_given_no_executable(mc, fake):
    fake()
    assert mc.lib().mc_replicate_constants(None, None, 0) == 1
    assert "not a GPU executable" in mc.lib().mc_last_error().decode()
