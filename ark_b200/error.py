"""Exception classes, one per status of the C ABI; names follow the reference
(ark/include/ark/error.hpp:29-43, python/ark/error.py)."""


class BaseError(Exception):
    pass


class InternalError(BaseError):
    pass


class InvalidUsageError(BaseError):
    pass


class ModelError(BaseError):
    pass


class PlanError(BaseError):
    pass


class UnsupportedError(BaseError):
    pass


class SystemError(BaseError):  # noqa: A001 - name kept from the reference
    pass


class GpuError(BaseError):
    pass


STATUS_TO_ERROR = {1: InternalError, 2: InvalidUsageError, 3: ModelError, 4: PlanError, 5: UnsupportedError,
                   6: SystemError, 7: GpuError}
