"""Name generator with Paddle's counter semantics (python/paddle/base/unique_name.py:41-52):
``generate("linear")`` yields ``linear_0``, ``linear_1`` ...; ``guard()`` swaps in a fresh
generator so that two models built under separate guards get identical parameter names."""
from __future__ import annotations

import collections
import contextlib


class UniqueNameGenerator:
    def __init__(self, prefix: str = ""):
        self.ids = collections.defaultdict(int)
        self.prefix = prefix

    def __call__(self, key: str) -> str:
        tmp = self.ids[key]
        self.ids[key] += 1
        return self.prefix + "_".join([key, str(tmp)])


generator = UniqueNameGenerator()


def generate(key: str) -> str:
    return generator(key)


def switch(new_generator=None):
    global generator
    old = generator
    generator = new_generator if new_generator is not None else UniqueNameGenerator()
    return old


@contextlib.contextmanager
def guard(new_generator=None):
    if isinstance(new_generator, str):
        new_generator = UniqueNameGenerator(new_generator)
    old = switch(new_generator)
    try:
        yield
    finally:
        switch(old)
