class B200Backend:
    name = "b200"


def install_into_upstream():
    raise NotImplementedError
