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


class AbstractExchange:
    """Interface of the point-to-point engines (src/AbstractExchange.hxx:7-23): what
    ``GaspiEx`` and ``Comprex`` / ``FastComprex`` have in common, so that code can be written
    against either."""

    def writeRemote(self, vector):
        raise NotImplementedError

    def readRemote(self, vector=None):
        raise NotImplementedError

    def readRemote_add(self, vector):
        raise NotImplementedError

    def connectTx(self, targRank: int, tag: int = 0):
        raise NotImplementedError

    def connectRx(self, srcRank: int, tag: int = 0):
        raise NotImplementedError

    def connectTo(self, srcRank: int, targRank: int, tag: int = 0):
        """srcRank: receive from this rank; targRank: send to this rank."""
        raise NotImplementedError
