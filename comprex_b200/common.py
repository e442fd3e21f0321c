"""Small mix-ins kept for interface parity with the reference (common.py:1-13)."""


class Gettable:
    """``get()`` hands the object itself to whoever needs the native handle."""

    def get(self):
        return self


Getable = Gettable  # the reference spells it both ways (ComprEx.py:158)


class Subscribable:
    """Keeps dependants alive for as long as the owner lives."""

    def __init__(self):
        self._subscribers = []

    def subscribe(self, obj) -> None:
        self._subscribers.append(obj)

    def unsubscribe(self, obj) -> None:
        if obj in self._subscribers:
            self._subscribers.remove(obj)
