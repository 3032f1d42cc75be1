"""``paddle.sysconfig``: include / library directories of the native components."""
import os

_ROOT = os.path.dirname(os.path.abspath(__file__))


def get_include():
    return os.path.join(_ROOT, "csrc", "kernels")


def get_lib():
    return os.path.join(_ROOT, "lib")
