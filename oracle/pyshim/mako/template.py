import re


class Template(object):
    """${expr} substitution where expr is a plain identifier passed to render()."""

    def __init__(self, text, **kwargs):
        self.text = text

    def render(self, **names):
        for line in self.text.splitlines():
            if line.lstrip().startswith("%") and not line.lstrip().startswith("%%"):
                raise NotImplementedError("mako control lines are not supported by this stand-in")

        def sub(m):
            key = m.group(1).strip()
            if key not in names:
                raise NameError(key)
            return str(names[key])
        return re.sub(r"\$\{([^}]*)\}", sub, self.text)
