"""Minimal stand-in: the reference only uses ``DefaultNamedArg`` in type hints."""


def DefaultNamedArg(type=None, name=None):  # noqa: A002,N802
    return type


def NamedArg(type=None, name=None):  # noqa: A002,N802
    return type


def DefaultArg(type=None, name=None):  # noqa: A002,N802
    return type


def Arg(type=None, name=None):  # noqa: A002,N802
    return type


def VarArg(type=None):  # noqa: A002,N802
    return type


def KwArg(type=None):  # noqa: A002,N802
    return type
