"""``fastfold`` import names on top of ``fastfold_b200``.

Programs written against the reference package keep working unchanged::

    from fastfold.distributed import init_dap
    from fastfold.model.fastnn import Evoformer, set_chunk_size
    from fastfold.model.hub import AlphaFold
    from fastfold.utils.inject_fastnn import inject_fastnn      # or: from fastfold.utils import inject_fastnn
    from fastfold.utils.import_weights import import_jax_weights_
    from fastfold.config import model_config

Every name resolves to the module of ``fastfold_b200`` that implements it (no code lives here).
"""
import importlib
import sys

VERSION = "0.2.0-b200"

_ALIASES = {
    "fastfold.config": "fastfold_b200.config",
    "fastfold.common": "fastfold_b200.common",
    "fastfold.common.residue_constants": "fastfold_b200.common.residue_constants",
    "fastfold.common.protein": "fastfold_b200.common.protein",
    "fastfold.distributed": "fastfold_b200.parallel",
    "fastfold.distributed.core": "fastfold_b200.parallel.core",
    "fastfold.distributed.comm": "fastfold_b200.parallel.comm",
    "fastfold.distributed.comm_async": "fastfold_b200.parallel.comm_async",
    "fastfold.model": "fastfold_b200.models",
    "fastfold.model.fastnn": "fastfold_b200.models.fastnn",
    "fastfold.model.fastnn.ops": "fastfold_b200.models.fastnn.ops",
    "fastfold.model.fastnn.msa": "fastfold_b200.models.fastnn.msa",
    "fastfold.model.fastnn.triangle": "fastfold_b200.models.fastnn.triangle",
    "fastfold.model.fastnn.evoformer": "fastfold_b200.models.fastnn.evoformer",
    "fastfold.model.fastnn.kernel": "fastfold_b200.ops.compat",
    # the reference's kernel back ends (Triton, CUDA extension, TorchScript) are one set of sm_100a kernels here
    "fastfold.model.fastnn.kernel.attention_core": "fastfold_b200.ops.attention",
    "fastfold.model.fastnn.kernel.softmax": "fastfold_b200.ops.softmax",
    "fastfold.model.fastnn.kernel.layer_norm": "fastfold_b200.ops.layer_norm",
    "fastfold.model.fastnn.kernel.jit": "fastfold_b200.ops.compat",
    "fastfold.model.fastnn.kernel.jit.fused_ops": "fastfold_b200.ops.fused_ops",
    "fastfold.model.fastnn.kernel.jit.options": "fastfold_b200.ops.compat",
    "fastfold.model.fastnn.kernel.triton": "fastfold_b200.ops.compat",
    "fastfold.model.fastnn.kernel.triton.attention_core": "fastfold_b200.ops.attention",
    "fastfold.model.fastnn.kernel.triton.softmax": "fastfold_b200.ops.softmax",
    "fastfold.model.fastnn.kernel.triton.layer_norm": "fastfold_b200.ops.layer_norm",
    "fastfold.model.fastnn.kernel.cuda_native": "fastfold_b200.ops.compat",
    "fastfold.model.fastnn.kernel.cuda_native.softmax": "fastfold_b200.ops.softmax",
    "fastfold.model.fastnn.kernel.cuda_native.layer_norm": "fastfold_b200.ops.layer_norm",
    "fastfold.model.nn": "fastfold_b200.models.nn",
    "fastfold.model.nn.primitives": "fastfold_b200.models.nn.primitives",
    "fastfold.model.nn.evoformer": "fastfold_b200.models.nn.evoformer",
    "fastfold.model.nn.structure_module": "fastfold_b200.models.nn.structure_module",
    "fastfold.model.nn.heads": "fastfold_b200.models.nn.heads",
    "fastfold.model.nn.embedders": "fastfold_b200.models.nn.embedders",
    "fastfold.model.nn.template": "fastfold_b200.models.nn.template",
    "fastfold.model.hub": "fastfold_b200.models.hub",
    "fastfold.model.hub.alphafold": "fastfold_b200.models.hub.alphafold",
    "fastfold.model.hub.loss": "fastfold_b200.models.hub.loss",
    "fastfold.model.hub.lr_scheduler": "fastfold_b200.models.hub.lr_scheduler",
    "fastfold.utils": "fastfold_b200.utils",
    "fastfold.utils.inject_fastnn": "fastfold_b200.utils.inject_fastnn",
    "fastfold.utils.import_weights": "fastfold_b200.utils.import_weights",
    "fastfold.utils.rigid_utils": "fastfold_b200.utils.rigid_utils",
    "fastfold.utils.feats": "fastfold_b200.utils.feats",
    "fastfold.utils.tensor_utils": "fastfold_b200.utils.tensor_utils",
    "fastfold.utils.checkpointing": "fastfold_b200.utils.checkpointing",
    "fastfold.utils.validation_utils": "fastfold_b200.utils.validation_utils",
    "fastfold.data": "fastfold_b200.data",
    "fastfold.data.data_pipeline": "fastfold_b200.data.data_pipeline",
    "fastfold.data.data_transforms": "fastfold_b200.data.data_transforms",
    "fastfold.data.parsers": "fastfold_b200.data.parsers",
    "fastfold.data.data_modules": "fastfold_b200.data.data_modules",
    "fastfold.data.data_transforms_multimer": "fastfold_b200.data.data_transforms_multimer",
    "fastfold.data.feature_pipeline": "fastfold_b200.data.feature_pipeline",
    "fastfold.data.input_pipeline": "fastfold_b200.data.input_pipeline",
    "fastfold.data.input_pipeline_multimer": "fastfold_b200.data.input_pipeline_multimer",
    "fastfold.data.feature_processing_multimer": "fastfold_b200.data.feature_processing_multimer",
    "fastfold.data.msa_pairing": "fastfold_b200.data.msa_pairing",
    "fastfold.data.msa_identifiers": "fastfold_b200.data.msa_identifiers",
    "fastfold.data.templates": "fastfold_b200.data.templates",
    "fastfold.data.mmcif_parsing": "fastfold_b200.data.mmcif_parsing",
    "fastfold.data.errors": "fastfold_b200.data.errors",
    "fastfold.data.tools": "fastfold_b200.data.tools",
    "fastfold.data.tools.jackhmmer": "fastfold_b200.data.tools.jackhmmer",
    "fastfold.data.tools.hhblits": "fastfold_b200.data.tools.hhblits",
    "fastfold.data.tools.hhsearch": "fastfold_b200.data.tools.hhsearch",
    "fastfold.data.tools.hmmsearch": "fastfold_b200.data.tools.hmmsearch",
    "fastfold.data.tools.hmmbuild": "fastfold_b200.data.tools.hmmbuild",
    "fastfold.data.tools.kalign": "fastfold_b200.data.tools.kalign",
    "fastfold.data.tools.utils": "fastfold_b200.data.tools.utils",
    "fastfold.workflow": "fastfold_b200.workflow",
    "fastfold.workflow.workflow_run": "fastfold_b200.workflow.workflow_run",
    "fastfold.workflow.factory": "fastfold_b200.workflow.factory",
    "fastfold.workflow.factory.task_factory": "fastfold_b200.workflow.factory.task_factory",
    "fastfold.workflow.factory.jackhmmer": "fastfold_b200.workflow.factory.jackhmmer",
    "fastfold.workflow.factory.hhblits": "fastfold_b200.workflow.factory.hhblits",
    "fastfold.workflow.factory.hhsearch": "fastfold_b200.workflow.factory.hhsearch",
    "fastfold.workflow.factory.hhfilter": "fastfold_b200.workflow.factory.hhfilter",
    "fastfold.workflow.factory.hmmsearch": "fastfold_b200.workflow.factory.hmmsearch",
    "fastfold.workflow.template": "fastfold_b200.workflow.template",
    "fastfold.workflow.template.fastfold_data_workflow": "fastfold_b200.workflow.template.fastfold_data_workflow",
    "fastfold.workflow.template.fastfold_multimer_data_workflow": "fastfold_b200.workflow.template.fastfold_multimer_data_workflow",
    "fastfold.relax": "fastfold_b200.relax",
    "fastfold.relax.relax": "fastfold_b200.relax.relax",
    "fastfold.relax.amber_minimize": "fastfold_b200.relax.amber_minimize",
    "fastfold.relax.cleanup": "fastfold_b200.relax.cleanup",
    "fastfold.relax.utils": "fastfold_b200.relax.utils",
    "fastfold.utils.all_atom_multimer": "fastfold_b200.utils.all_atom_multimer",
    "fastfold.utils.superimposition": "fastfold_b200.utils.superimposition",
    "fastfold.utils.test_utils": "fastfold_b200.utils.test_utils",
    "fastfold.utils.geometry": "fastfold_b200.utils.geometry",
    "fastfold.utils.geometry.vector": "fastfold_b200.utils.geometry",
    "fastfold.utils.geometry.rotation_matrix": "fastfold_b200.utils.geometry",
    "fastfold.utils.geometry.rigid_matrix_vector": "fastfold_b200.utils.geometry",
    "fastfold.utils.geometry.quat_rigid": "fastfold_b200.utils.geometry",
    "fastfold.utils.geometry.utils": "fastfold_b200.utils.geometry",
    "fastfold.utils.geometry.test_utils": "fastfold_b200.utils.geometry",
    "fastfold.model.fastnn.template": "fastfold_b200.models.fastnn.template",
    "fastfold.model.fastnn.embedders": "fastfold_b200.models.fastnn.embedders",
    "fastfold.model.fastnn.embedders_multimer": "fastfold_b200.models.fastnn.embedders_multimer",
    "fastfold.model.fastnn.initializer": "fastfold_b200.models.fastnn.initializer",
    "fastfold.model.nn.embedders_multimer": "fastfold_b200.models.nn.embedders_multimer",
}

# modules of the OpenFold-layout model that the reference splits over more files than this package does
_ALIASES.update({
    "fastfold.model.nn.msa": "fastfold_b200.models.nn.msa",
    "fastfold.model.nn.dropout": "fastfold_b200.models.nn.dropout",
    "fastfold.model.nn.pair_transition": "fastfold_b200.models.nn.pair",
    "fastfold.model.nn.outer_product_mean": "fastfold_b200.models.nn.pair",
    "fastfold.model.nn.triangular_attention": "fastfold_b200.models.nn.pair",
    "fastfold.model.nn.triangular_multiplicative_update": "fastfold_b200.models.nn.pair",
})


class _AliasFinder:
    """Import hook: ``fastfold.x.y`` -> the aliased ``fastfold_b200`` module object."""

    @staticmethod
    def find_spec(name, path=None, target=None):
        if name in _ALIASES:
            from importlib.machinery import ModuleSpec
            return ModuleSpec(name, _AliasLoader(), is_package=True)
        return None


class _AliasLoader:
    @staticmethod
    def create_module(spec):
        mod = importlib.import_module(_ALIASES[spec.name])
        return mod

    @staticmethod
    def exec_module(module):
        pass


if not any(isinstance(f, type) and f.__name__ == "_AliasFinder" for f in sys.meta_path):
    sys.meta_path.insert(0, _AliasFinder)
