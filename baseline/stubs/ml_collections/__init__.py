"""Stand-in for the ``ml_collections`` package (not installed here), covering what the reference's ``fastfold/config.py``
uses: ``ConfigDict`` with attribute access over nested dicts and ``FieldReference`` cells shared between several
fields (assigning to any of the fields updates the cell, so every field that shares it follows)."""
import copy as _copy


class FieldReference:
    def __init__(self, default, field_type=None, op=None, required=False):
        self._value = default
        self._field_type = field_type

    def get(self):
        return self._value

    def set(self, value, type_safe=True):
        self._value = value.get() if isinstance(value, FieldReference) else value

    def empty(self):
        return self._value is None


def _wrap(v):
    if isinstance(v, dict) and not isinstance(v, ConfigDict):
        return ConfigDict(v)
    return v


class ConfigDict:
    def __init__(self, initial_dictionary=None, type_safe=True, convert_dict=True, **kwargs):
        object.__setattr__(self, "_fields", {})
        object.__setattr__(self, "_locked", False)
        src = dict(initial_dictionary or {})
        src.update(kwargs)
        for k, v in src.items():
            self._fields[k] = _wrap(v)

    # -- mapping protocol ----------------------------------------------------
    def __getitem__(self, key):
        v = self._fields[key]
        return v.get() if isinstance(v, FieldReference) else v

    def __setitem__(self, key, value):
        cur = self._fields.get(key)
        if isinstance(cur, FieldReference) and not isinstance(value, FieldReference):
            cur.set(value)
        else:
            self._fields[key] = _wrap(value)

    def __getattr__(self, key):
        if key.startswith("__"):
            raise AttributeError(key)
        try:
            return self[key]
        except KeyError:
            raise AttributeError(key)

    def __setattr__(self, key, value):
        self[key] = value

    def __delitem__(self, key):
        del self._fields[key]

    def __contains__(self, key):
        return key in self._fields

    def __iter__(self):
        return iter(self._fields)

    def __len__(self):
        return len(self._fields)

    def keys(self):
        return self._fields.keys()

    def values(self):
        return [self[k] for k in self._fields]

    def items(self, preserve_field_references=False):
        return [(k, self._fields[k] if preserve_field_references else self[k]) for k in self._fields]

    def get(self, key, default=None):
        return self[key] if key in self._fields else default

    def get_ref(self, key):
        v = self._fields[key]
        if not isinstance(v, FieldReference):
            v = FieldReference(v)
            self._fields[key] = v
        return v

    def update(self, *other, **kwargs):
        for o in other:
            for k, v in (o.items() if hasattr(o, "items") else o):
                if k in self._fields and isinstance(self._fields[k], ConfigDict) and isinstance(v, (dict, ConfigDict)):
                    self._fields[k].update(v)
                else:
                    self[k] = v
        for k, v in kwargs.items():
            self[k] = v

    def to_dict(self, visit_map=None, preserve_field_references=False):
        return {k: (v.to_dict() if isinstance(v, ConfigDict) else v) for k, v in self.items()}

    def copy_and_resolve_references(self, visit_map=None):
        return ConfigDict(self.to_dict())

    def lock(self):
        object.__setattr__(self, "_locked", True)
        return self

    def unlock(self):
        object.__setattr__(self, "_locked", False)
        return self

    def unlocked(self):
        import contextlib
        return contextlib.nullcontext(self)

    def __deepcopy__(self, memo):
        new = ConfigDict()
        memo[id(self)] = new
        for k, v in self._fields.items():
            new._fields[k] = _copy.deepcopy(v, memo)      # the memo keeps shared FieldReference cells shared
        return new

    def __repr__(self):
        return "ConfigDict(%r)" % (self.to_dict(),)

    def __eq__(self, other):
        return isinstance(other, ConfigDict) and self.to_dict() == other.to_dict()


FrozenConfigDict = ConfigDict
