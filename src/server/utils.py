from allie_b200.serve.server import SYSTEMS, System, recv_dict, send_dict  # noqa: F401
