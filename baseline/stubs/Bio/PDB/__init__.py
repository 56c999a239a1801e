class PDBParser:
    def __init__(self, *args, **kwargs):
        raise RuntimeError("BioPython is not installed; this stand-in only satisfies the import")
