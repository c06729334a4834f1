"""Error kinds and process exit codes.

The kinds and the codes follow the reference's error type
(crates/vipera-errors/src/lib.rs:12-47 for the kinds, :94-104 for the codes):
1 usage, 2 bad input (io, parse, unsupported, invalid argument), 3 infeasible,
4 internal.
"""


class ViperaError(Exception):
    """Base of every error this package raises on purpose."""

    exit_code = 4
    kind = "internal"


class UsageError(ViperaError):
    """The command line was wrong (unknown flag, missing argument)."""

    exit_code = 1
    kind = "usage"


class IoError(ViperaError):
    """A file could not be read or written."""

    exit_code = 2
    kind = "io"


class ParseError(ViperaError):
    """A file was read but its contents are malformed."""

    exit_code = 2
    kind = "parse"

    def __init__(self, message, offset=None):
        super().__init__(message if offset is None else f"{message} (at byte {offset})")
        self.offset = offset


class UnsupportedError(ViperaError):
    """The input is well formed but asks for something this engine does not build."""

    exit_code = 2
    kind = "unsupported"


class InvalidArgumentError(ViperaError):
    """A value handed to the API is outside what it accepts."""

    exit_code = 2
    kind = "invalid_argument"


class InfeasibleError(ViperaError):
    """The request cannot fit (cache pages, device memory)."""

    exit_code = 3
    kind = "infeasible"


class InternalError(ViperaError):
    """A fault of the engine itself (a kernel reported an error, a missing build)."""

    exit_code = 4
    kind = "internal"
