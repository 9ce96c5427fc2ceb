"""Error types mirroring the candle errors this path can raise."""


class CandleError(RuntimeError):
    """candle::Error::Msg -- the message strings are the ones candle uses (`candle::bail!`)."""


class InvalidIndex(CandleError, IndexError):
    """candle::Error::InvalidIndex { index, size, op } (candle-core/src/cpu_backend/mod.rs:539-546)."""

    def __init__(self, index: int, size: int, op: str = "index-select", position: int | None = None):
        super().__init__(f"{op} invalid index {index} with dim size {size}")  # candle-core/src/error.rs:129
        self.index, self.size, self.op, self.position = index, size, op, position
