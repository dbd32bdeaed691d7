from .modeling_bert import (BertEmbeddings, BertIntermediate, BertOutput, BertAttention, BertLayer, SequencePool, BertEncoder,
                            BertModel, BertModelNoPooler, PoolingType, BertPooler)
from .qmodeling_bert import QBertIntermediate, QBertOutput, QBertLayer, QBertEncoder, QBertModel
from .modules import MultiHeadedAttention, PositionwiseFeedForward
from .modeling_gpt2 import GPT2Model
from .modeling_decoder import TransformerDecoderLayer, TransformerDecoder
from .modeling_smart_pad import (MultiHeadedAttentionSmartBatch, BertLayerSmartBatch, BertEncoderSmartBatch, BertModelSmartBatch,
                                 BertModelNoPoolerSmartBatch)
from .modeling_distillbert import DistillBertAttention, DistrillFFN, DistrillTransformerBlock, DistrillTransformer, DistilBertModel
from .modeling_roberta import RobertaModel
from .modeling_albert import AlbertAttention, AlbertLayer, AlbertLayerGroup, AlbertTransformer, AlbertModel
from .return_type import ReturnType

__all__ = ['BertEmbeddings', 'BertIntermediate', 'BertOutput', 'BertAttention', 'BertLayer', 'BertEncoder', 'BertModel',
           'BertModelNoPooler', 'ReturnType', 'BertPooler', 'SequencePool', 'PoolingType', 'MultiHeadedAttention',
           'PositionwiseFeedForward', 'QBertIntermediate', 'QBertOutput', 'QBertLayer', 'QBertEncoder', 'QBertModel', 'GPT2Model',
           'MultiHeadedAttentionSmartBatch', 'BertLayerSmartBatch', 'BertEncoderSmartBatch', 'BertModelSmartBatch',
           'BertModelNoPoolerSmartBatch', 'DistillBertAttention', 'DistrillFFN', 'DistrillTransformerBlock', 'DistrillTransformer',
           'DistilBertModel', 'RobertaModel', 'AlbertAttention', 'AlbertLayer', 'AlbertLayerGroup', 'AlbertTransformer', 'AlbertModel', 'TransformerDecoderLayer', 'TransformerDecoder']
