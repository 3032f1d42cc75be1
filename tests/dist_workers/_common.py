import os
import pickle
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def dump(obj):
    out = os.environ["PD_TEST_OUT"]
    rank = int(os.environ.get("PADDLE_TRAINER_ID", "0"))
    with open(f"{out}.{rank}", "wb") as f:
        pickle.dump(obj, f)
