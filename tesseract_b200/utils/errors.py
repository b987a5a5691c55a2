"""Error types with the reference's names (include/tesseract/utils/Logging.hpp:12-63)."""


class TesseractError(RuntimeError):
    pass


class ShapeError(TesseractError):
    pass


class DeviceError(TesseractError):
    pass


def check(cond: bool, msg: str, *fmt, exc=TesseractError) -> None:
    """TESSERACT_CHECK: raise ``exc`` with a formatted message when ``cond`` is false."""
    if not cond:
        raise exc(msg.format(*fmt) if fmt else msg)
