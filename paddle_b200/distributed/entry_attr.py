"""Sparse-table entry policies (python/paddle/distributed/entry_attr.py): attribute strings consumed by
``static.nn.sparse_embedding``."""


class EntryAttr:
    def __init__(self):
        self._name = None

    def _to_attr(self):
        raise NotImplementedError("EntryAttr is base class")


class ProbabilityEntry(EntryAttr):
    def __init__(self, probability):
        super().__init__()
        if not isinstance(probability, float):
            raise ValueError("probability must be a float in (0,1)")
        if probability <= 0 or probability >= 1:
            raise ValueError("probability must be a float in (0,1)")
        self._name, self._probability = "probability_entry", probability

    def _to_attr(self):
        return ":".join([self._name, str(self._probability)])


class CountFilterEntry(EntryAttr):
    def __init__(self, count_filter):
        super().__init__()
        if not isinstance(count_filter, int):
            raise ValueError("count_filter must be a valid integer greater than 0")
        if count_filter < 0:
            raise ValueError("count_filter must be a valid integer greater or equal than 0")
        self._name, self._count_filter = "count_filter_entry", count_filter

    def _to_attr(self):
        return ":".join([self._name, str(self._count_filter)])


class ShowClickEntry(EntryAttr):
    def __init__(self, show_name, click_name):
        super().__init__()
        if not isinstance(show_name, str) or not isinstance(click_name, str):
            raise ValueError("show_name click_name must be a str")
        self._name, self._show_name, self._click_name = "show_click_entry", show_name, click_name

    def _to_attr(self):
        return ":".join([self._name, self._show_name, self._click_name])
