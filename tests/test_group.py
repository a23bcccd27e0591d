"""The NCCL group of the C ABI with NCCL replaced by fakes (no GPU, no NCCL needed).

Failure detection is exercised on the host only: a communicator that never completes (a rank that
never arrives), an NCCL call that fails, and two thread "ranks" of which one stays away. The
library must answer with a status within its time limit, abort the communicator and never hang.
"""
import ctypes
import threading
import time

from ishizuki_b200 import _lib

NCCL_SUCCESS, NCCL_SYSTEM_ERROR, NCCL_IN_PROGRESS = 0, 2, 7


class UniqueId(ctypes.Structure):
    _fields_ = [("internal", ctypes.c_char * 128)]


GET_ID = ctypes.CFUNCTYPE(ctypes.c_int, ctypes.POINTER(UniqueId))
INIT = ctypes.CFUNCTYPE(ctypes.c_int, ctypes.POINTER(ctypes.c_void_p), ctypes.c_int, UniqueId, ctypes.c_int, ctypes.c_void_p)
ASYNC = ctypes.CFUNCTYPE(ctypes.c_int, ctypes.c_void_p, ctypes.POINTER(ctypes.c_int))
GATHER = ctypes.CFUNCTYPE(ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_void_p,
                          ctypes.c_void_p)
COMM = ctypes.CFUNCTYPE(ctypes.c_int, ctypes.c_void_p)
ERRSTR = ctypes.CFUNCTYPE(ctypes.c_void_p, ctypes.c_int)


class Api(ctypes.Structure):
    _fields_ = [("get_unique_id", GET_ID), ("init", INIT), ("async_error", ASYNC), ("all_gather", GATHER),
                ("abort", COMM), ("destroy", COMM), ("error_string", ERRSTR)]


class FakeNccl:
    """A communicator is 'complete' once `needed` ranks have called init; init_result and
    state_result let a test make calls fail."""

    def __init__(self, needed: int, init_result: int = NCCL_IN_PROGRESS):
        self.needed, self.init_result = needed, init_result
        self.joined, self.aborted, self.destroyed = 0, 0, 0
        self.lock = threading.Lock()
        self._strings = {code: ctypes.create_string_buffer(text) for code, text in
                         ((NCCL_SYSTEM_ERROR, b"unhandled system error (fake)"), (NCCL_SUCCESS, b"no error"), (-1, b"error"))}

        def get_id(out):
            out[0].internal = b"fake-id"
            return NCCL_SUCCESS

        def init(comm, world, uid, rank, cfg):
            if self.init_result not in (NCCL_SUCCESS, NCCL_IN_PROGRESS):
                return self.init_result
            with self.lock:
                self.joined += 1
            comm[0] = 0x1000 + rank
            return self.init_result

        def async_error(comm, state):
            with self.lock:
                state[0] = NCCL_SUCCESS if self.joined >= self.needed else NCCL_IN_PROGRESS
            return NCCL_SUCCESS

        def gather(send, recv, count, dtype, comm, stream):
            return NCCL_SUCCESS

        def abort(comm):
            with self.lock:
                self.aborted += 1
            return NCCL_SUCCESS

        def destroy(comm):
            with self.lock:
                self.destroyed += 1
            return NCCL_SUCCESS

        def error_string(code):
            return ctypes.cast(self._strings.get(code, self._strings[-1]), ctypes.c_void_p).value

        self.table = Api(GET_ID(get_id), INIT(init), ASYNC(async_error), GATHER(gather), COMM(abort), COMM(destroy),
                         ERRSTR(error_string))

    def __enter__(self):
        assert _lib.load().ishi_group_debug_set_api(ctypes.byref(self.table)) == _lib.OK
        return self

    def __exit__(self, *exc):
        _lib.load().ishi_group_debug_set_api(None)


def create(rank: int, world: int, timeout_ms: int):
    lib = _lib.load()
    uid = ctypes.create_string_buffer(_lib.GROUP_ID_BYTES)
    assert lib.ishi_group_unique_id(uid) == _lib.OK
    handle = ctypes.c_void_p()
    rc = lib.ishi_group_create(uid, rank, world, timeout_ms, ctypes.byref(handle))
    return rc, handle


def test_a_rank_that_never_arrives_times_out_and_the_communicator_is_aborted():
    lib = _lib.load()
    with FakeNccl(needed=2) as fake:
        t0 = time.time()
        rc, handle = create(0, 2, 200)
        took = time.time() - t0
        assert rc == _lib.E_TIMEOUT and 0.15 < took < 5.0
        assert fake.aborted == 1
        assert b"aborted" in lib.ishi_group_last_error(handle)
        # a broken group refuses work instead of touching NCCL again
        assert lib.ishi_projection_apply_sharded(handle, None, None, 8, None, None) == _lib.E_INVALID
        lib.ishi_group_destroy(handle)
        assert fake.destroyed == 0


def test_an_nccl_failure_is_reported_with_its_message():
    lib = _lib.load()
    with FakeNccl(needed=1, init_result=NCCL_SYSTEM_ERROR):
        rc, handle = create(0, 2, 200)
        assert rc == _lib.E_NCCL
        assert b"system error" in lib.ishi_group_last_error(handle)
        lib.ishi_group_destroy(handle)


def test_two_thread_ranks_meet_and_one_staying_away_is_noticed():
    lib = _lib.load()
    with FakeNccl(needed=2) as fake:
        results = {}

        def rank_main(r):
            results[r] = create(r, 2, 2000)

        threads = [threading.Thread(target=rank_main, args=(r,)) for r in range(2)]
        threads[0].start()
        time.sleep(0.1)  # rank 1 is late, not absent
        threads[1].start()
        for t in threads:
            t.join()
        assert [results[r][0] for r in range(2)] == [_lib.OK, _lib.OK]
        for r in range(2):
            lib.ishi_group_destroy(results[r][1])
        assert fake.destroyed == 2 and fake.aborted == 0
    with FakeNccl(needed=3) as fake:  # three expected, two come
        results = {}
        threads = [threading.Thread(target=lambda r=r: results.__setitem__(r, create(r, 3, 300))) for r in range(2)]
        for t in threads:
            t.start()
        for t in threads:
            t.join()
        assert [results[r][0] for r in range(2)] == [_lib.E_TIMEOUT, _lib.E_TIMEOUT]
        for r in range(2):
            lib.ishi_group_destroy(results[r][1])


def test_arguments_are_checked_before_nccl_is_touched():
    lib = _lib.load()
    with FakeNccl(needed=1) as fake:
        uid = ctypes.create_string_buffer(_lib.GROUP_ID_BYTES)
        handle = ctypes.c_void_p()
        assert lib.ishi_group_create(uid, 2, 2, 100, ctypes.byref(handle)) == _lib.E_INVALID
        assert lib.ishi_group_create(uid, 0, 9, 100, ctypes.byref(handle)) == _lib.E_INVALID
        assert lib.ishi_group_create(None, 0, 1, 100, ctypes.byref(handle)) == _lib.E_INVALID
        assert fake.joined == 0
