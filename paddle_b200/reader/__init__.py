"""Reader decorators (python/paddle/reader/decorator.py): a *reader* is a zero-argument callable returning an
iterable of samples; decorators compose readers into new readers."""
from __future__ import annotations

import itertools
import queue
import random
import threading

__all__ = []


def cache(reader):
    all_data = tuple(reader())

    def cached():
        yield from all_data
    return cached


def map_readers(func, *readers):
    def reader():
        yield from map(func, *[r() for r in readers])
    return reader


def shuffle(reader, buf_size):
    def shuffled():
        buf = []
        for e in reader():
            buf.append(e)
            if len(buf) >= buf_size:
                random.shuffle(buf)
                yield from buf
                buf = []
        random.shuffle(buf)
        yield from buf
    return shuffled


def chain(*readers):
    def reader():
        return itertools.chain(*[r() for r in readers])
    return reader


class ComposeNotAligned(ValueError):
    pass


def compose(*readers, **kwargs):
    check_alignment = kwargs.pop("check_alignment", True)

    def tup(x):
        return x if isinstance(x, tuple) else (x,)

    def reader():
        its = [r() for r in readers]
        if not check_alignment:
            for outs in zip(*its):
                yield sum(map(tup, outs), ())
        else:
            for outs in itertools.zip_longest(*its):
                if any(o is None for o in outs):
                    raise ComposeNotAligned("outputs of readers are not aligned.")
                yield sum(map(tup, outs), ())
    return reader


def buffered(reader, size):
    end = object()

    def fill(q):
        for d in reader():
            q.put(d)
        q.put(end)

    def buffered_reader():
        q = queue.Queue(maxsize=size)
        t = threading.Thread(target=fill, args=(q,), daemon=True)
        t.start()
        while True:
            e = q.get()
            if e is end:
                return
            yield e
    return buffered_reader


def firstn(reader, n):
    def firstn_reader():
        yield from itertools.islice(reader(), n)
    return firstn_reader


def xmap_readers(mapper, reader, process_num, buffer_size, order=False):
    """Maps samples with ``process_num`` worker threads; ``order`` keeps the input order."""
    from concurrent.futures import ThreadPoolExecutor

    def xreader():
        with ThreadPoolExecutor(process_num) as pool:
            if order:
                yield from pool.map(mapper, reader())
            else:
                pending = set()
                import concurrent.futures as cf
                for s in reader():
                    pending.add(pool.submit(mapper, s))
                    if len(pending) >= buffer_size:
                        done, pending = cf.wait(pending, return_when=cf.FIRST_COMPLETED)
                        for d in done:
                            yield d.result()
                for d in cf.as_completed(pending):
                    yield d.result()
    return xreader


def multiprocess_reader(readers, use_pipe=True, queue_size=1000):
    """Runs every reader in its own thread and interleaves their samples (the reference forks processes; the
    samples and their order guarantees — none across readers — are the same)."""
    end = object()

    def reader():
        q = queue.Queue(queue_size)

        def work(r):
            for s in r():
                q.put(s)
            q.put(end)
        for r in readers:
            threading.Thread(target=work, args=(r,), daemon=True).start()
        left = len(readers)
        while left:
            s = q.get()
            if s is end:
                left -= 1
            else:
                yield s
    return reader


# the functions live in ``paddle.reader.decorator`` in the reference
from .._core.submodule_alias import alias_submodules as _alias  # noqa: E402
_alias(__name__, ("decorator",))
