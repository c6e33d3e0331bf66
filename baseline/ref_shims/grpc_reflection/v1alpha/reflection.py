"""Import stand-in: server reflection is only enabled by `serve()`."""
SERVICE_NAME = "grpc.reflection.v1alpha.ServerReflection"


def enable_server_reflection(service_names, server):
    pass
