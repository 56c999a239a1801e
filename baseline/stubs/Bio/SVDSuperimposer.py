"""Stand-in for ``Bio.SVDSuperimposer`` (BioPython is not installed): least-squares superposition of two point sets by
singular value decomposition, with BioPython's method names.  Used only by the reference package's
``fastfold/utils/superimposition.py`` when that package runs as a baseline / oracle."""
import numpy as np


class SVDSuperimposer:
    def __init__(self):
        self.reference_coords = self.coords = self.transformed_coords = self.rot = self.tran = self.rms = None

    def set(self, reference_coords, coords):
        reference_coords, coords = np.asarray(reference_coords, dtype=np.float64), np.asarray(coords, dtype=np.float64)
        if reference_coords.shape != coords.shape or coords.ndim != 2:
            raise ValueError("Coordinate number/dimension mismatch.")
        self.reference_coords, self.coords = reference_coords, coords
        self.transformed_coords = self.rot = self.tran = self.rms = None

    def run(self):
        if self.coords is None:
            raise ValueError("No coordinates set.")
        centre_moving, centre_fixed = self.coords.mean(axis=0), self.reference_coords.mean(axis=0)
        u, _, vt = np.linalg.svd((self.coords - centre_moving).T @ (self.reference_coords - centre_fixed))
        rot = u @ vt                                   # row vectors: transformed = coords @ rot + tran
        if np.linalg.det(rot) < 0:                     # a reflection: flip the axis of the smallest singular value
            vt[2] = -vt[2]
            rot = u @ vt
        self.rot, self.tran = rot, centre_fixed - centre_moving @ rot

    def get_transformed(self):
        if self.rot is None:
            raise ValueError("Nothing superimposed yet.")
        if self.transformed_coords is None:
            self.transformed_coords = self.coords @ self.rot + self.tran
        return self.transformed_coords

    def get_rotran(self):
        if self.rot is None:
            raise ValueError("Nothing superimposed yet.")
        return self.rot, self.tran

    def get_init_rms(self):
        return float(np.sqrt(((self.coords - self.reference_coords) ** 2).sum() / self.coords.shape[0]))

    def get_rms(self):
        if self.rms is None:
            diff = self.get_transformed() - self.reference_coords
            self.rms = float(np.sqrt((diff ** 2).sum() / self.coords.shape[0]))
        return self.rms
