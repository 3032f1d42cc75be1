"""Throughput timer of the training loop (python/paddle/profiler/timer.py:20-420): reader cost, batch cost and
instances per second, averaged between two ``step_info`` calls and over the whole run.  ``benchmark()`` returns the
process-wide instance; the data loader reports to it through ``before_reader`` / ``after_reader`` and the profiler
through ``begin`` / ``step`` / ``end``."""
from __future__ import annotations

import time


class Stack:
    """The benchmark keeps one ``Event`` per nested ``DataLoader`` iteration (an evaluation loop inside training)."""

    def __init__(self):
        self.items = []

    def push(self, item):
        self.items.append(item)

    def pop(self):
        return self.items.pop() if self.items else None

    def peek(self):
        return self.items[-1] if self.items else None

    def is_empty(self):
        return not self.items

    def size(self):
        return len(self.items)


class TimeAverager:
    def __init__(self):
        self.reset()

    def reset(self):
        self._total_iters = 0
        self._total_time = 0.0
        self._total_samples = 0

    def record(self, usetime, num_samples=None):
        self._total_iters += 1
        self._total_time += usetime
        if num_samples:
            self._total_samples += num_samples

    def get_average(self):
        return self._total_time / self._total_iters if self._total_iters else 0.0

    def get_ips_average(self):
        if not self._total_time:
            return 0.0
        return (self._total_samples or self._total_iters) / self._total_time


class Event:
    """Accumulators of one loop: since the last report (``*_averager``) and since its start (``total_*``); the
    first ``skip_iter`` steps are left out of the run totals as warm-up."""

    def __init__(self):
        self.reader_cost_averager = TimeAverager()
        self.batch_cost_averager = TimeAverager()
        self.total_samples = 0
        self.total_iters = 0
        self.skip_iter = 10
        self.reader_records = dict(max=0.0, min=float("inf"), total=0.0)
        self.batch_records = dict(max=0.0, min=float("inf"), total=0.0)
        self.speed_records = dict(max=0.0, min=float("inf"))
        self.reader = None
        self.need_record = True
        self.speed_mode = "samples/s"
        self.speed_unit = "samples/s"

    def reset(self):
        self.reader_cost_averager.reset()
        self.batch_cost_averager.reset()

    def record_reader(self, usetime):
        self.reader_cost_averager.record(usetime)
        if self.total_iters >= self.skip_iter:
            self._update(self.reader_records, usetime)

    def record_batch(self, usetime, num_samples=None):
        self.batch_cost_averager.record(usetime, num_samples)
        self.total_iters += 1
        if self.total_iters > self.skip_iter:
            self._update(self.batch_records, usetime)
            if num_samples:
                self.total_samples += num_samples
                speed = num_samples / usetime if usetime else 0.0
            else:
                speed = 1.0 / usetime if usetime else 0.0
            self.speed_records["max"] = max(self.speed_records["max"], speed)
            self.speed_records["min"] = min(self.speed_records["min"], speed)

    @staticmethod
    def _update(rec, v):
        rec["max"], rec["min"], rec["total"] = max(rec["max"], v), min(rec["min"], v), rec["total"] + v

    def reader_average(self):
        return self.reader_cost_averager.get_average()

    def batch_average(self):
        return self.batch_cost_averager.get_average()

    def speed_average(self):
        return self.batch_cost_averager.get_ips_average()

    def get_summary(self):
        n = self.total_iters - self.skip_iter
        if n <= 0:
            return None
        reader_avg = self.reader_records["total"] / n
        batch_avg = self.batch_records["total"] / n
        ips = (self.total_samples / self.batch_records["total"]) if self.total_samples and self.batch_records["total"] else \
            (n / self.batch_records["total"] if self.batch_records["total"] else 0.0)
        return dict(reader_summary=dict(avg=reader_avg, max=self.reader_records["max"], min=self.reader_records["min"]),
                    batch_summary=dict(avg=batch_avg, max=self.batch_records["max"], min=self.batch_records["min"]),
                    ips_summary=dict(avg=ips, max=self.speed_records["max"], min=self.speed_records["min"]),
                    reader_ratio=100.0 * reader_avg / batch_avg if batch_avg else 0.0, steps=n)


class Hook:
    def begin(self, benchmark): ...
    def end(self, benchmark): ...
    def before_reader(self, benchmark): ...
    def after_reader(self, benchmark): ...
    def after_step(self, benchmark): ...


class TimerHook(Hook):
    """Takes the wall-clock stamps.  No device synchronisation: the costs are those the host sees, as in the
    reference, so that the timer never slows the loop it measures."""

    def __init__(self):
        self.start_time = time.perf_counter()
        self.start_reader = time.perf_counter()

    def begin(self, benchmark):
        self.start_time = self.start_reader = time.perf_counter()

    def before_reader(self, benchmark):
        self.start_reader = time.perf_counter()

    def after_reader(self, benchmark):
        ev = benchmark.current_event
        if ev is None or not ev.need_record:
            return
        ev.record_reader(time.perf_counter() - self.start_reader)

    def after_step(self, benchmark):
        ev = benchmark.current_event
        if ev is None or not ev.need_record:
            return
        now = time.perf_counter()
        ev.record_batch(now - self.start_time, benchmark.num_samples)
        self.start_time = now

    def end(self, benchmark):
        ev = benchmark.current_event
        if ev is None:
            return
        summary = ev.get_summary()
        if summary is None:
            return
        benchmark.last_summary = summary
        if benchmark.print_summary:
            print(benchmark.format_summary(summary, ev.speed_unit))


class Benchmark:
    def __init__(self):
        self.num_samples = None
        self.hooks = {"timer_hook": TimerHook()}
        self.current_event = None
        self.events = Stack()
        self.print_summary = False
        self.last_summary = None

    def step(self, num_samples=None):
        self.num_samples = num_samples
        self.after_step()

    def step_info(self, unit=None):
        ev = self.current_event
        if ev is None:
            return ""
        unit = unit or ("samples" if ev.batch_cost_averager._total_samples else "steps")
        msg = ""
        if ev.reader_cost_averager._total_iters:
            msg += f"reader_cost: {ev.reader_average():.5f} s "
        msg += f"batch_cost: {ev.batch_average():.5f} s ips: {ev.speed_average():.3f} {unit}/s"
        ev.speed_unit = f"{unit}/s"
        ev.reset()
        return msg

    def begin(self):
        if self.current_event is None:
            self.current_event = Event()
            self.events.push(self.current_event)
        for h in self.hooks.values():
            h.begin(self)

    def before_reader(self):
        for h in self.hooks.values():
            h.before_reader(self)

    def after_reader(self):
        for h in self.hooks.values():
            h.after_reader(self)

    def after_step(self):
        for h in self.hooks.values():
            h.after_step(self)

    def end(self):
        for h in self.hooks.values():
            h.end(self)
        self.events.pop()
        self.current_event = self.events.peek()

    def check_if_need_record(self, reader):
        """A nested loader (evaluation inside training) gets its own event; only the loader that opened the current
        event reports into it."""
        if self.current_event is None:
            return
        if self.current_event.reader is None:
            self.current_event.reader = reader
        elif self.current_event.reader is not reader:
            self.current_event = Event()
            self.current_event.reader = reader
            self.events.push(self.current_event)

    @staticmethod
    def format_summary(summary, unit="samples/s"):
        r, b, i = summary["reader_summary"], summary["batch_summary"], summary["ips_summary"]
        rows = [("reader_cost (s)", r), ("batch_cost (s)", b), (f"ips ({unit})", i)]
        out = [f"Perf Summary over {summary['steps']} steps (reader share {summary['reader_ratio']:.2f} %)",
               f"{'':<18}{'avg':>12}{'max':>12}{'min':>12}"]
        out += [f"{n:<18}{v['avg']:>12.5f}{v['max']:>12.5f}{v['min']:>12.5f}" for n, v in rows]
        return "\n".join(out)


_benchmark = Benchmark()


def benchmark():
    return _benchmark
