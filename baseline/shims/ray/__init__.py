"""Import-time stand-in for `ray` (not installable here: no index, not in the offline wheel directory).  The
reference imports it while importing its config package (`aspec/transfer/mooncake/utils.py:34`); the model, loss
and optimizer path that the benchmark's reference arm runs starts no actor.  Decorators pass classes through
unchanged; anything that would start or talk to a cluster raises."""


def remote(*args, **kwargs):
    if len(args) == 1 and callable(args[0]) and not kwargs:
        return args[0]
    return lambda obj: obj


def _unavailable(*args, **kwargs):
    raise RuntimeError("ray is not installed; only the import is satisfied")


init = get = put = wait = kill = shutdown = get_actor = nodes = cluster_resources = available_resources = _unavailable


def is_initialized() -> bool:
    return False


class ObjectRef:
    pass


class _Namespace:
    def __getattr__(self, name):
        return _unavailable


actor = _Namespace()
exceptions = type("exceptions", (), {"RayActorError": RuntimeError, "RayTaskError": RuntimeError, "GetTimeoutError": TimeoutError,
                                     "RayError": RuntimeError, "ActorDiedError": RuntimeError})
