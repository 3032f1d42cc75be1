import os
import pickle
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def dump(obj, teardown=True):
    """Write this rank's results and leave.  Every worker calls this last.  The process groups are taken down in step
    (barrier, then destroy) and the process ends without running static destructors: with gloo, worker threads that
    are still parked in a collective's transport when the interpreter unloads have ended runs with ``terminate called
    without an active exception`` after the results were already written.  ``teardown=False`` skips the barrier for
    workers whose peers are gone on purpose."""
    out = os.environ["PD_TEST_OUT"]
    rank = int(os.environ.get("PADDLE_TRAINER_ID", "0"))
    with open(f"{out}.{rank}", "wb") as f:
        pickle.dump(obj, f)
        f.flush()
        os.fsync(f.fileno())
    try:
        import torch.distributed as tdist
        if teardown and tdist.is_initialized():
            tdist.barrier()
            tdist.destroy_process_group()
    except Exception:  # noqa: BLE001 - the results are on disk; teardown problems must not fail the rank
        pass
    sys.stdout.flush()
    sys.stderr.flush()
    os._exit(0)
