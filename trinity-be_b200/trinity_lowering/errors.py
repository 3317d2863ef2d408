"""Exception types of the runtime (names and fields as in the reference's errors module)."""


class RuntimeFailure(RuntimeError):
    """A call into a compiled plan, the driver or a completion wait failed.

    ``domain`` / ``stage`` / ``code`` / ``submitted`` / ``cleanup_domain`` / ``cleanup_code`` carry
    the artifact ABI's ErrorInfo; ``submitted`` tells whether GPU work may be in flight."""

    def __init__(self, message, domain=0, stage=0, code=0, submitted=False, cleanup_domain=0,
                 cleanup_code=0):
        super().__init__(message)
        self.domain, self.stage, self.code = domain, stage, code
        self.submitted = bool(submitted)
        self.cleanup_domain, self.cleanup_code = cleanup_domain, cleanup_code


class ResourceBusy(RuntimeError):
    """The object is in use: live children, pending work on another stream, or graph-owned."""


class DistributedFailure(RuntimeError):
    """A multi-rank step failed on some rank; the world is terminal afterwards."""


class CompileError(RuntimeError):
    """Building an artifact failed; ``diagnostics`` holds compiler, arguments, exit code, output."""

    def __init__(self, message, diagnostics=None):
        super().__init__(message)
        self.diagnostics = diagnostics
