"""Import stand-in: base classes of the gRPC server interceptors (the benchmark drives the model
runner directly, no gRPC server is started)."""


class AsyncServerInterceptor:
    pass


class ServerInterceptor:
    pass
