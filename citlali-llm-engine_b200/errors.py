"""One exception type and one precondition helper, used everywhere.

Mirrors ``citlali::Error`` / ``require()`` of the reference
(include/citlali/common.h:8-17).
"""


class CitlaliError(RuntimeError):
    """Every error the library raises on purpose."""


def require(condition, message):
    if not condition:
        raise CitlaliError(message() if callable(message) else message)
