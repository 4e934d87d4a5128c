"""SynBioS: synthetic-biography knowledge storage / extraction study on the MoE language model.

A client of the training system: it generates data, calls the shared shard writer, trains through ``scripts/train.py``
and then evaluates, probes and analyses the exported ``model.pt`` through ``MiniTransformer.hidden_states`` and the
router modules (reference: experiments/synbios_moe/).
"""
