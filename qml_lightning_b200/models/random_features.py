"""``RandomFourrierFeaturesModel``: dense random Fourier feature model (upstream qml_lightning/models/random_features.py)."""
import numpy as np
import torch

from .kernel import BaseKernel


class RandomFourrierFeaturesModel(BaseKernel, torch.nn.Module):

    def __init__(self, rep=None, elements=np.array([1, 6, 7, 8]), sigma=2.0, llambda=1e-10, nstacks=8192, npcas=128,
                 nbatch_train=64, nbatch_test=64):
        super(RandomFourrierFeaturesModel, self).__init__(rep, npcas, elements, sigma, llambda)
        self.device = rep.device
        self.npcas = npcas
        self.nbatch_train = nbatch_train
        self.nbatch_test = nbatch_test
        self._nfeatures = nstacks * self.npcas
        self.species = torch.from_numpy(np.asarray(elements)).float().to(self.device)
        self.sample_elemental_basis()
        self.feature_normalisation = np.sqrt(2.0 / self._nfeatures)
        self.alpha = None
        self.is_trained = False

    def sample_elemental_basis(self):
        """W ~ N(0,1)/(2 sigma^2), b ~ U(0, 2 pi) per element (upstream :42-55)."""
        D, d = self.nfeatures(), self.npcas
        self.W = torch.zeros((len(self.elements), d, D), dtype=torch.float32, device=self.device)
        self.b = torch.zeros((len(self.elements), D), dtype=torch.float32, device=self.device)
        for e in self.elements:
            idx = int(self.element2index[int(e)])
            self.W[idx] = torch.from_numpy(np.random.normal(0.0, 1.0, [d, D]) / (2 * self.sigma ** 2)).float().to(self.device)
            self.b[idx] = torch.from_numpy(np.random.uniform(0.0, 1.0, [D]) * 2.0 * np.pi).float().to(self.device)

    def nfeatures(self):
        return self._nfeatures
