from fairseq2_b200.assets.card import AssetCard, AssetCardError, AssetCardFieldNotFoundError
from fairseq2_b200.assets.download_manager import AssetDownloadError, AssetDownloadManager
from fairseq2_b200.assets.store import (AssetMetadataError, AssetMetadataProvider, AssetNotFoundError, AssetStore,
                                        FileAssetMetadataProvider, InMemoryAssetMetadataProvider, get_asset_store,
                                        register_checkpoint_models)
