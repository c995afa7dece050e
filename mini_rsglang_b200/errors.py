"""Error kinds of the engine, after the reference's `Error` enum
(crates/core/src/lib.rs:9-21): a request that is wrong in itself, a request that does not
fit, a failure below the engine, and use after shutdown."""


class EngineError(Exception):
    """Base of every error the engine raises on purpose."""


class InvalidRequest(EngineError):
    """The request, configuration or checkpoint is wrong in itself (`Error::Invalid`)."""


class CapacityError(EngineError):
    """The request is valid but does not fit the pool or the queue (`Error::Capacity`)."""


class BackendError(EngineError):
    """A device, kernel or build failure (`Error::Backend`)."""


class EngineStopped(EngineError):
    """The engine was shut down or failed earlier (`Error::Stopped`)."""
