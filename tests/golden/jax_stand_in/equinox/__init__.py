"""Just enough of equinox for the reference's BlockMask: a Module is a dataclass, a field is a dataclass field."""
import dataclasses


class Module:
    def __init_subclass__(cls, **kw):
        super().__init_subclass__(**kw)
        dataclasses.dataclass(eq=False)(cls)


def field(static=False, **kw):
    return dataclasses.field(**kw)
