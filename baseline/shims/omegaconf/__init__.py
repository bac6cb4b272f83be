"""Import-time stand-in for the `omegaconf` package, which is not installable here (no index, not in the offline
wheel directory).  The reference imports it at package import (`aspec/config/train_config.py:30`) for YAML
recipes only; the model, loss and optimizer code that the reference arm of the benchmark runs never calls into
it.  Any attempt to actually use it raises, so it cannot silently change behaviour."""


class _Unavailable:
    def __init__(self, *args, **kwargs):
        raise RuntimeError("omegaconf is not installed; only the import is satisfied")


class DictConfig(_Unavailable):
    pass


class ListConfig(_Unavailable):
    pass


class OmegaConf:
    def __getattr__(self, name):
        raise RuntimeError("omegaconf is not installed; only the import is satisfied")

    @staticmethod
    def register_new_resolver(*args, **kwargs):
        return None


MISSING = "???"
