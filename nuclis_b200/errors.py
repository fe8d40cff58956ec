"""Status codes of the C ABI (``nu_status`` in include/nuclis_cuda.h) as an exception."""

STATUS_NAMES = {
    0: "Ok",
    1: "UnsupportedTensorEncoding",
    2: "InvalidRowLength",
    3: "InvalidByteLength",
    4: "InvalidShape",
    5: "MergeDeclined",
    6: "NotRecording",
    7: "AlreadyRecording",
    8: "BufferFailed",
    9: "ExecutionFailed",
    10: "InitializationFailed",
    11: "CommFailed",
    12: "TooLarge",
}


class NuclisError(Exception):
    """A failed call; ``name`` is the reference's error name (e.g. ``InvalidShape``)."""

    def __init__(self, status: int, message: str = ""):
        self.status = status
        self.name = STATUS_NAMES.get(status, f"status {status}")
        super().__init__(f"{self.name}: {message}" if message else self.name)
